"""egg_c_b200 — ctypes host binding of libegg_b200.so (the C ABI of include/egg_b200.h).

The library is the product; this module only loads it, mirrors `struct egg_config`
and wraps each entry point so that tests and bench.py read like the reference's
training loop (full_cuda_train_transformer_adam_mgpu.cu:1506-1688).  There is no
CPU fallback: a missing or unloadable library raises.
"""
import ctypes as C
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libegg_b200.so")

EGG_OK, EGG_E_INVALID, EGG_E_CUDA, EGG_E_NOMEM, EGG_E_TIMEOUT, EGG_E_NCCL, EGG_E_STATE = 0, -1, -2, -3, -4, -5, -6

EXPORTS = [
    "egg_config_defaults", "egg_config_validate", "egg_model_bytes", "egg_opt_state_bytes", "egg_ctx_create",
    "egg_ctx_destroy", "egg_last_error", "egg_sync", "egg_upload_model", "egg_download_model", "egg_upload_opt_state",
    "egg_download_opt_state", "egg_set_dataset", "egg_set_dataset_tokens", "egg_eval_chunk", "egg_read_losses", "egg_compute_fitness_pairs",
    "egg_write_fitness", "egg_read_fitness", "egg_nccl_unique_id", "egg_comm_init", "egg_allgather_fitness", "egg_set_update_sharding", "egg_update_owner_plan",
    "egg_apply_update", "egg_generation_host", "egg_perturbed_projection", "egg_update_reconstruct", "egg_update_matrix",
    "egg_update_reconstruct_noalloc", "egg_scales_bytes", "egg_upload_scales", "egg_download_scales", "egg_set_overlay_steps",
    "egg_timer_start", "egg_timer_stop", "egg_profile_enable", "egg_profile_read", "egg_profile_name", "egg_launch_count",
    "egg_wave_members", "egg_set_fused_epilogues", "egg_fused_epilogues_active", "egg_set_attention_tensor_core", "egg_measure_int8_peak", "egg_selftest_index_math", "egg_generate", "egg_save_checkpoint", "egg_load_checkpoint", "egg_wire_fixed_bytes", "egg_wire_encode", "egg_wire_decode_header", "egg_wire_decode_body",
    "egg_ternary_packed_size", "egg_ternary_pack", "egg_ternary_unpack", "egg_deggs_chunk_fitness", "egg_next_seed",
    "egg_gru_config_defaults", "egg_gru_model_bytes", "egg_gru_state_bytes", "egg_gru_create", "egg_gru_destroy",
    "egg_gru_upload_model", "egg_gru_download_model", "egg_gru_upload_states", "egg_gru_download_states", "egg_gru_set_dataset",
    "egg_gru_generation", "egg_gru_launch_count",
    "egg_learning_rate", "egg_worker_options_defaults", "egg_worker_run", "egg_worker_engine_from_ctx", "egg_get_config",
    "egg_log_open", "egg_log_record", "egg_log_close",
]
EGG_PROF_N = 16


class EggConfig(C.Structure):
    """struct egg_config (include/egg_b200.h)."""
    _fields_ = [(n, C.c_int32) for n in (
        "hidden_dim", "head_dim", "n_layers", "seq_len", "vocab_size", "population_size",
        "fixed_point", "sigma_shift", "sigma_shift_vector", "shift_attn", "shift_out",
        "shift_logit", "shift_mlp_up", "shift_mlp_down", "softmax_scale_bit", "rope_scale_bit",
        "device_mask", "device_gaussian", "host_mask", "use_same_data", "use_muon",
        "chunk_relative_loss")] + [
        ("softmax_exp_scale", C.c_double), ("adam_beta1", C.c_float), ("adam_beta2", C.c_float),
        ("adam_eps", C.c_float), ("adam_weight_decay", C.c_float), ("muon_momentum", C.c_float),
        ("muon_lr_scale", C.c_float), ("ntt_mode", C.c_int32)]


class GruConfig(C.Structure):
    """struct egg_gru_config: the #defines of full_trained_egg.c:10-21."""
    _fields_ = [(n, C.c_int32) for n in ("hidden_dim", "n_layers", "vocab_size", "seq_len", "population_size",
                                          "fixed_point", "sigma_shift", "update_threshold")]


class WireMsg(C.Structure):
    """struct egg_wire_msg."""
    _fields_ = [("opcode", C.c_int32), ("payload_size", C.c_uint32), ("seed", C.c_uint64), ("last_step", C.c_uint64),
                ("data_position", C.c_uint64), ("updates_count", C.c_uint64), ("sum_loss", C.c_int64)]


EVAL_CHUNK_FN = C.CFUNCTYPE(C.c_int, C.c_void_p, C.c_uint32, C.c_int64, C.c_int, C.c_int, C.POINTER(C.c_int32))
APPLY_UPDATE_FN = C.CFUNCTYPE(C.c_int, C.c_void_p, C.POINTER(C.c_int32), C.c_int, C.c_uint32, C.c_float, C.c_float, C.POINTER(C.c_uint64))
GENERATE_FN = C.CFUNCTYPE(C.c_int, C.c_void_p, C.c_int64, C.c_uint32, C.c_char_p, C.c_int)
BEFORE_RESULT_FN = C.CFUNCTYPE(C.c_int, C.c_void_p, C.c_int64, C.c_int)


class WorkerEngine(C.Structure):
    """Mirror of struct egg_worker_engine."""
    _fields_ = [("self", C.c_void_p), ("eval_chunk", EVAL_CHUNK_FN), ("apply_update", APPLY_UPDATE_FN), ("generate", GENERATE_FN)]


class WorkerOptions(C.Structure):
    """Mirror of struct egg_worker_options."""
    _fields_ = [("host", C.c_char * 64), ("port", C.c_int), ("population_size", C.c_int), ("chunk_size", C.c_int),
                ("initial_seed", C.c_uint64), ("wait_sleep_ms", C.c_int), ("recv_timeout_ms", C.c_int), ("generate_every", C.c_int),
                ("mean_filter", C.c_int), ("mean_exponent", C.c_double), ("adaptive_threshold", C.c_int), ("threshold_alpha", C.c_double),
                ("stop_at_step", C.c_int64), ("max_requests", C.c_int64), ("stop_flag", C.POINTER(C.c_int)),
                ("before_result", BEFORE_RESULT_FN), ("hook_self", C.c_void_p)]


class WorkerStats(C.Structure):
    """Mirror of struct egg_worker_stats."""
    _fields_ = [(n, C.c_uint64) for n in ("requests", "chunks_done", "updates_applied", "waits", "results_dropped", "bytes_sent",
                                          "bytes_received", "final_step", "final_seed")]


class EggError(RuntimeError):
    def __init__(self, code, msg):
        super().__init__("egg_b200 error %d: %s" % (code, msg))
        self.code = code


_lib = None


def build(force=False):
    import importlib.util
    spec = importlib.util.spec_from_file_location("egg_c_b200_build", os.path.join(_HERE, "build.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod.build(force=force)


def lib():
    """Loads libegg_b200.so; raises if it is missing (there is no fallback path)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise EggError(EGG_E_STATE, "libegg_b200.so is not built (run python egg.c_b200/build.py)")
        L = C.CDLL(LIB_PATH)
        P = C.POINTER
        cfgp = P(EggConfig)
        vp = C.c_void_p
        L.egg_config_defaults.argtypes = [cfgp]
        L.egg_config_defaults.restype = None
        L.egg_config_validate.argtypes = [cfgp, P(C.c_char_p)]
        L.egg_model_bytes.argtypes = [cfgp]
        L.egg_model_bytes.restype = C.c_int64
        L.egg_opt_state_bytes.argtypes = [cfgp]
        L.egg_opt_state_bytes.restype = C.c_int64
        gcp = P(GruConfig)
        L.egg_gru_config_defaults.argtypes = [gcp]
        L.egg_gru_config_defaults.restype = None
        for f in (L.egg_gru_model_bytes, L.egg_gru_state_bytes):
            f.argtypes = [gcp]
            f.restype = C.c_int64
        L.egg_gru_create.argtypes = [gcp, C.c_int, P(vp)]
        L.egg_gru_destroy.argtypes = [vp]
        L.egg_gru_destroy.restype = None
        for f in (L.egg_gru_upload_model, L.egg_gru_download_model, L.egg_gru_upload_states, L.egg_gru_download_states,
                  L.egg_gru_set_dataset):
            f.argtypes = [vp, vp, C.c_int64]
        L.egg_gru_generation.argtypes = [vp, C.c_uint32, C.c_int64, C.c_int, C.c_int, vp, vp]
        L.egg_gru_launch_count.argtypes = [vp]
        L.egg_gru_launch_count.restype = C.c_int64
        L.egg_measure_int8_peak.argtypes = [vp, C.c_int, C.c_int, C.c_int, C.c_int, P(C.c_double)]
        L.egg_generate.argtypes = [vp, vp, C.c_int, C.c_int, C.c_uint32, C.c_float, C.c_float, C.c_float]
        L.egg_save_checkpoint.argtypes = [vp, C.c_char_p, C.c_int64]
        L.egg_load_checkpoint.argtypes = [vp, C.c_char_p, C.c_char_p]
        L.egg_scales_bytes.argtypes = [cfgp]
        L.egg_scales_bytes.restype = C.c_int64
        L.egg_set_overlay_steps.argtypes = [C.c_void_p, C.c_int, C.c_int]
        L.egg_ctx_create.argtypes = [cfgp, C.c_int, C.c_int, P(vp)]
        L.egg_ctx_destroy.argtypes = [vp]
        L.egg_ctx_destroy.restype = None
        L.egg_last_error.restype = C.c_char_p
        L.egg_sync.argtypes = [vp]
        for f in (L.egg_upload_model, L.egg_download_model, L.egg_upload_opt_state, L.egg_download_opt_state, L.egg_set_dataset,
                  L.egg_set_dataset_tokens, L.egg_upload_scales, L.egg_download_scales):
            f.argtypes = [vp, vp, C.c_int64]
        L.egg_eval_chunk.argtypes = [vp, C.c_uint32, C.c_int64, C.c_int, C.c_int]
        L.egg_read_losses.argtypes = [vp, vp, C.c_int, C.c_int]
        L.egg_compute_fitness_pairs.argtypes = [vp, C.c_int, C.c_int]
        L.egg_write_fitness.argtypes = [vp, vp, C.c_int, C.c_int]
        L.egg_read_fitness.argtypes = [vp, vp, C.c_int, C.c_int]
        L.egg_nccl_unique_id.argtypes = [vp]
        L.egg_comm_init.argtypes = [vp, vp, C.c_int, C.c_int]
        L.egg_allgather_fitness.argtypes = [vp]
        L.egg_set_update_sharding.argtypes = [vp, C.c_int]
        L.egg_update_owner_plan.argtypes = [vp, C.c_int, vp, vp, vp, vp, C.c_int]
        L.egg_apply_update.argtypes = [vp, C.c_uint32, C.c_float, P(C.c_uint64)]
        L.egg_generation_host.argtypes = [vp, vp, C.c_int64, C.c_int64, C.c_uint32, C.c_float, vp, P(C.c_uint64)]
        L.egg_perturbed_projection.argtypes = [vp, vp, vp, vp, C.c_int64, C.c_int, C.c_int, C.c_int, C.c_uint32, C.c_int,
                                               C.c_int, C.c_int, C.c_int, C.c_int]
        L.egg_update_reconstruct.argtypes = [vp, vp, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_uint32, vp, C.c_int]
        L.egg_update_matrix.argtypes = [vp, vp, vp, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, vp, C.c_int, C.c_uint32, C.c_float, C.c_int,
                                        C.c_int, P(C.c_uint64)]
        L.egg_update_reconstruct_noalloc.argtypes = [vp, vp, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_uint32, C.c_int, vp]
        L.egg_timer_start.argtypes = [vp]
        L.egg_timer_stop.argtypes = [vp, P(C.c_float)]
        L.egg_profile_enable.argtypes = [vp, C.c_int]
        L.egg_profile_read.argtypes = [vp, P(C.c_float), P(C.c_int64)]
        L.egg_profile_name.argtypes = [C.c_int]
        L.egg_profile_name.restype = C.c_char_p
        L.egg_launch_count.argtypes = [vp]
        L.egg_launch_count.restype = C.c_int64
        L.egg_wave_members.argtypes = [vp]
        L.egg_set_fused_epilogues.argtypes = [vp, C.c_int]
        L.egg_fused_epilogues_active.argtypes = [vp]
        L.egg_set_attention_tensor_core.argtypes = [vp, C.c_int]
        L.egg_learning_rate.argtypes = [C.c_int64]
        L.egg_learning_rate.restype = C.c_float
        L.egg_worker_options_defaults.argtypes = [P(WorkerOptions)]
        L.egg_worker_options_defaults.restype = None
        L.egg_worker_run.argtypes = [P(WorkerOptions), P(WorkerEngine), P(WorkerStats)]
        L.egg_worker_engine_from_ctx.argtypes = [vp, P(WorkerEngine)]
        L.egg_get_config.argtypes = [vp, P(EggConfig)]
        L.egg_log_open.argtypes = [C.c_char_p, P(EggConfig), C.c_int, C.c_uint64, P(vp)]
        L.egg_log_record.argtypes = [vp, C.c_int64, C.c_double, C.c_uint64, C.c_float]
        L.egg_log_close.argtypes = [vp]
        L.egg_log_close.restype = None
        L.egg_wire_fixed_bytes.argtypes = [C.c_int]
        L.egg_wire_encode.argtypes = [P(WireMsg), vp, C.c_int]
        L.egg_wire_decode_header.argtypes = [vp, P(C.c_int), P(C.c_uint32)]
        L.egg_wire_decode_body.argtypes = [C.c_int, vp, C.c_int, P(WireMsg)]
        L.egg_ternary_packed_size.argtypes = [C.c_int64]
        L.egg_ternary_packed_size.restype = C.c_int64
        L.egg_ternary_pack.argtypes = [vp, C.c_int64, vp]
        L.egg_ternary_pack.restype = None
        L.egg_ternary_unpack.argtypes = [vp, C.c_int64, vp]
        L.egg_ternary_unpack.restype = None
        L.egg_deggs_chunk_fitness.argtypes = [vp, C.c_int, C.c_int, C.c_double, C.c_int, C.c_double, vp, P(C.c_int64)]
        L.egg_next_seed.argtypes = [C.c_uint32, C.c_uint64]
        L.egg_next_seed.restype = C.c_uint32
        _lib = L
    return _lib


def _check(rc):
    if rc != 0:
        raise EggError(rc, lib().egg_last_error().decode())


def default_config(**kw):
    cfg = EggConfig()
    lib().egg_config_defaults(C.byref(cfg))
    for k, v in kw.items():
        if not hasattr(cfg, k):
            raise KeyError(k)
        setattr(cfg, k, v)
    return cfg


def update_owner_plan(cfg, world, spans=False):
    """(owners, costs) of every parameter as the sharded update deals them over `world` ranks (no GPU needed); with
    spans=True also the byte offset inside the model and the number of weights of every parameter."""
    n = lib().egg_update_owner_plan(C.byref(cfg), world, None, None, None, None, 0)
    _check(min(n, 0))
    owners, costs, offs, lens = np.zeros(n, np.int32), np.zeros(n, np.int64), np.zeros(n, np.int64), np.zeros(n, np.int64)
    _check(min(lib().egg_update_owner_plan(C.byref(cfg), world, _ptr(owners), _ptr(costs), _ptr(offs), _ptr(lens), n), 0))
    return (owners, costs, offs, lens) if spans else (owners, costs)


def model_bytes(cfg):
    return lib().egg_model_bytes(C.byref(cfg))


def default_gru_config(**kw):
    cfg = GruConfig()
    lib().egg_gru_config_defaults(C.byref(cfg))
    for k, v in kw.items():
        if not hasattr(cfg, k):
            raise KeyError(k)
        setattr(cfg, k, v)
    return cfg


def gru_model_bytes(gcfg):
    return lib().egg_gru_model_bytes(C.byref(gcfg))


def gru_state_bytes(gcfg):
    return lib().egg_gru_state_bytes(C.byref(gcfg))


def opt_state_bytes(cfg):
    return lib().egg_opt_state_bytes(C.byref(cfg))


def selftest_index_math():
    """Host-only check of the multiply-shift division shared by host and kernels (raises on a mismatch)."""
    L = lib()
    L.egg_selftest_index_math.argtypes = []
    L.egg_selftest_index_math.restype = C.c_int
    _check(L.egg_selftest_index_math())


def scales_bytes(cfg):
    return lib().egg_scales_bytes(C.byref(cfg))


def _ptr(a):
    if a is None:
        return None
    if isinstance(a, int):
        return C.c_void_p(a)
    return a.ctypes.data_as(C.c_void_p)


class Context:
    """One egg_ctx: one process, one GPU."""

    def __init__(self, cfg, device=0, wave_members=0):
        self.cfg = cfg
        self._h = C.c_void_p()
        _check(lib().egg_ctx_create(C.byref(cfg), device, wave_members, C.byref(self._h)))

    def close(self):
        if self._h:
            lib().egg_ctx_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def sync(self):
        _check(lib().egg_sync(self._h))

    def upload_model(self, model):
        model = np.ascontiguousarray(model, np.int8)
        _check(lib().egg_upload_model(self._h, _ptr(model), model.nbytes))

    def download_model(self):
        out = np.zeros(model_bytes(self.cfg), np.int8)
        _check(lib().egg_download_model(self._h, _ptr(out), out.nbytes))
        return out

    def upload_opt_state(self, state):
        state = np.ascontiguousarray(state, np.uint8)
        _check(lib().egg_upload_opt_state(self._h, _ptr(state), state.nbytes))

    def download_opt_state(self):
        out = np.zeros(opt_state_bytes(self.cfg), np.uint8)
        _check(lib().egg_download_opt_state(self._h, _ptr(out), out.nbytes))
        return out

    def upload_scales(self, scales):
        """AdaptiveScales bytes (d-eggs adaptive-noise overlays); None switches back to unscaled noise."""
        if scales is None:
            _check(lib().egg_upload_scales(self._h, None, 0))
            return
        scales = np.ascontiguousarray(scales, np.int8)
        _check(lib().egg_upload_scales(self._h, _ptr(scales), scales.nbytes))

    def download_scales(self):
        out = np.zeros(scales_bytes(self.cfg), np.int8)
        _check(lib().egg_download_scales(self._h, _ptr(out), out.nbytes))
        return out

    def set_overlay_steps(self, inc, dec):
        _check(lib().egg_set_overlay_steps(self._h, inc, dec))

    def generate(self, seed_tokens, gen_len, seed, temp=1.0, min_p=0.0, penalty=0.0):
        """Returns the seed tokens followed by gen_len sampled ones (uint8)."""
        buf = np.zeros(len(seed_tokens) + gen_len, np.uint8)
        buf[:len(seed_tokens)] = seed_tokens
        _check(lib().egg_generate(self._h, _ptr(buf), len(seed_tokens), gen_len, seed & 0xFFFFFFFF, temp, min_p, penalty))
        return buf

    def save_checkpoint(self, directory, step):
        _check(lib().egg_save_checkpoint(self._h, os.fsencode(directory), step))

    def load_checkpoint(self, model_path, adam_path=None):
        _check(lib().egg_load_checkpoint(self._h, os.fsencode(model_path), os.fsencode(adam_path) if adam_path else None))

    def measure_int8_peak(self, m=16384, n=2048, k=2048, iters=20):
        """1e12 int8 ops/s of the GEMM's TMA + tcgen05 loop alone (accumulators dropped, operands in L2)."""
        t = C.c_double(0)
        _check(lib().egg_measure_int8_peak(self._h, m, n, k, iters, C.byref(t)))
        return t.value

    def set_dataset(self, tokens):
        """Byte tokens at vocab_size 256; uint32 tokens (the reference's TokenType of its tokenizer build) otherwise."""
        if self.cfg.vocab_size == 256:
            tokens = np.ascontiguousarray(tokens, np.uint8)
            _check(lib().egg_set_dataset(self._h, _ptr(tokens), len(tokens)))
        else:
            tokens = np.ascontiguousarray(tokens, np.uint32)
            _check(lib().egg_set_dataset_tokens(self._h, _ptr(tokens), len(tokens)))

    def eval_chunk(self, step_seed, start_idx, pop_offset, count):
        _check(lib().egg_eval_chunk(self._h, step_seed & 0xFFFFFFFF, start_idx, pop_offset, count))

    def read_losses(self, offset, count):
        out = np.zeros(count, np.int32)
        _check(lib().egg_read_losses(self._h, _ptr(out), offset, count))
        return out

    def compute_fitness_pairs(self, pair_offset, pair_count):
        _check(lib().egg_compute_fitness_pairs(self._h, pair_offset, pair_count))

    def write_fitness(self, fit, pair_offset=0):
        fit = np.ascontiguousarray(fit, np.int32)
        _check(lib().egg_write_fitness(self._h, _ptr(fit), pair_offset, len(fit)))

    def read_fitness(self, pair_offset, pair_count):
        out = np.zeros(pair_count, np.int32)
        _check(lib().egg_read_fitness(self._h, _ptr(out), pair_offset, pair_count))
        return out

    def comm_init(self, id128, rank, world):
        buf = (C.c_char * 128).from_buffer_copy(bytes(id128))
        _check(lib().egg_comm_init(self._h, buf, rank, world))

    def set_update_sharding(self, enable=True):
        """Each parameter is updated by one rank and broadcast (needs comm_init); download_opt_state becomes a collective."""
        _check(lib().egg_set_update_sharding(self._h, 1 if enable else 0))

    def allgather_fitness(self):
        _check(lib().egg_allgather_fitness(self._h))

    def apply_update(self, step_seed, lr):
        n = C.c_uint64(0)
        _check(lib().egg_apply_update(self._h, step_seed & 0xFFFFFFFF, C.c_float(lr), C.byref(n)))
        return n.value

    def generation_host(self, tokens, step, step_seed, lr, losses_out=None):
        """tokens: pinned/pageable host array (uint8, or uint32 when vocab_size != 256) or None to keep the resident dataset."""
        n = C.c_uint64(0)
        if tokens is not None:
            assert tokens.dtype == (np.uint8 if self.cfg.vocab_size == 256 else np.uint32), "token width does not match vocab_size"
        tp, tl = (None, 0) if tokens is None else (_ptr(tokens), len(tokens))
        _check(lib().egg_generation_host(self._h, tp, tl, step, step_seed & 0xFFFFFFFF, C.c_float(lr), _ptr(losses_out), C.byref(n)))
        return n.value

    def perturbed_projection(self, x, w_packed, y, rows, k_dim, n_dim, rows_per_member, seed, off_a, off_b,
                             rank1_shift, out_shift, on_device=False):
        _check(lib().egg_perturbed_projection(self._h, _ptr(x), _ptr(w_packed), _ptr(y), rows, k_dim, n_dim, rows_per_member,
                                              seed & 0xFFFFFFFF, off_a, off_b, rank1_shift, out_shift, 1 if on_device else 0))

    def update_reconstruct(self, fitness, pairs, rows_k, cols_n, off_a, off_b, seed_base, step_seed, vote_out, on_device=False):
        _check(lib().egg_update_reconstruct(self._h, _ptr(fitness), pairs, rows_k, cols_n, off_a, off_b, seed_base,
                                            step_seed & 0xFFFFFFFF, _ptr(vote_out), 1 if on_device else 0))


    def update_matrix(self, d_w_packed, d_opt_state, rows_k, cols_n, off_a, off_b, seed_base, d_fitness, pairs, step_seed, lr,
                      optimizer=0, split=False):
        """Device pointers; one AdamW (optimizer 0) or Muon (1) update of one matrix in place. Returns the number of changed weights."""
        n = C.c_uint64(0)
        _check(lib().egg_update_matrix(self._h, _ptr(d_w_packed), _ptr(d_opt_state), rows_k, cols_n, off_a, off_b, seed_base,
                                       _ptr(d_fitness), pairs, step_seed & 0xFFFFFFFF, C.c_float(lr), optimizer, 1 if split else 0,
                                       C.byref(n)))
        return n.value

    def update_reconstruct_noalloc(self, d_fitness, pairs, rows_k, cols_n, off_a, off_b, seed_base, step_seed, split, d_vote_out):
        """Device pointers in and out; uses the library's built-in operand buffer, allocates nothing."""
        _check(lib().egg_update_reconstruct_noalloc(self._h, _ptr(d_fitness), pairs, rows_k, cols_n, off_a, off_b, seed_base,
                                                    step_seed & 0xFFFFFFFF, 1 if split else 0, _ptr(d_vote_out)))

    def timer_start(self):
        _check(lib().egg_timer_start(self._h))

    def timer_stop(self):
        ms = C.c_float(0)
        _check(lib().egg_timer_stop(self._h, C.byref(ms)))
        return ms.value

    def profile_enable(self, on=True):
        _check(lib().egg_profile_enable(self._h, 1 if on else 0))

    def profile_read(self):
        """{class name: (milliseconds, launches)} since the last read."""
        ms = (C.c_float * EGG_PROF_N)()
        n = (C.c_int64 * EGG_PROF_N)()
        _check(lib().egg_profile_read(self._h, ms, n))
        return {lib().egg_profile_name(i).decode(): (ms[i], n[i]) for i in range(EGG_PROF_N)}

    def launch_count(self):
        return lib().egg_launch_count(self._h)

    def set_fused_epilogues(self, level):
        """0 / False: two-kernel adaptive norms; 1 / True: row-owning projections; 2 (the default of a new context):
        also the next mean-abs norm inside the MLP-down epilogue; 3: LN2 inside the output projection as well (slower on B200)."""
        _check(lib().egg_set_fused_epilogues(self._h, int(level)))

    def set_attention_tensor_core(self, mode):
        """0 / False: the mma.sync kernel; 1 / True: scores and weighted sums on tcgen05; 2: scores on mma.sync, weighted
        sums on tcgen05 with the accumulators in tensor memory."""
        _check(lib().egg_set_attention_tensor_core(self._h, int(mode)))

    def fused_epilogues_active(self):
        """The level in effect (0 when the configuration takes the two-kernel form)."""
        return int(lib().egg_fused_epilogues_active(self._h))

    def wave_members(self):
        return lib().egg_wave_members(self._h)


def nccl_unique_id():
    buf = (C.c_char * 128)()
    _check(lib().egg_nccl_unique_id(buf))
    return bytes(buf)


# ---- d-eggs worker boundary (host side) ----
def wire_encode(msg):
    buf = (C.c_uint8 * 64)()
    n = lib().egg_wire_encode(C.byref(msg), buf, 64)
    if n < 0:
        raise EggError(n, "cannot encode wire message")
    return bytes(buf[:n])


def wire_decode(data):
    """(WireMsg, total_len) of an encoded header + fixed body."""
    raw = (C.c_uint8 * len(data)).from_buffer_copy(data)
    op, total = C.c_int(0), C.c_uint32(0)
    rc = lib().egg_wire_decode_header(raw, C.byref(op), C.byref(total))
    if rc:
        raise EggError(rc, "bad wire header")
    msg = WireMsg()
    body = (C.c_uint8 * (len(data) - 10)).from_buffer_copy(data[10:])
    rc = lib().egg_wire_decode_body(op.value, body, len(data) - 10, C.byref(msg))
    if rc:
        raise EggError(rc, "bad wire body")
    return msg, total.value


def ternary_pack(values):
    values = np.ascontiguousarray(values, np.int32)
    out = np.zeros(lib().egg_ternary_packed_size(len(values)), np.uint8)
    lib().egg_ternary_pack(_ptr(values), len(values), _ptr(out))
    return out


def ternary_unpack(packed, count):
    packed = np.ascontiguousarray(packed, np.uint8)
    out = np.zeros(count, np.int32)
    lib().egg_ternary_unpack(_ptr(packed), count, _ptr(out))
    return out


def deggs_chunk_fitness(losses, mean_filter=1, exponent=1.2, adaptive=1, alpha=0.1):
    losses = np.ascontiguousarray(losses, np.int32)
    fit = np.zeros(len(losses) // 2, np.int32)
    sl = C.c_int64(0)
    _check(lib().egg_deggs_chunk_fitness(_ptr(losses), len(losses), mean_filter, exponent, adaptive, alpha, _ptr(fit), C.byref(sl)))
    return fit, sl.value


def next_seed(seed, step):
    return lib().egg_next_seed(seed & 0xFFFFFFFF, step)


def learning_rate(step):
    return float(lib().egg_learning_rate(step))


def worker_options(**kw):
    o = WorkerOptions()
    lib().egg_worker_options_defaults(C.byref(o))
    for k, v in kw.items():
        if k == "host":
            v = v.encode()
        setattr(o, k, v)
    return o


def worker_run(options, engine):
    """Runs the d-eggs worker loop until one of its stop conditions; returns (return code, WorkerStats).  The call
    releases the GIL, so several workers can run in threads of one process; callbacks of a Python engine take it back."""
    st = WorkerStats()
    rc = lib().egg_worker_run(C.byref(options), C.byref(engine), C.byref(st))
    return rc, st


def worker_engine_from_ctx(ctx):
    e = WorkerEngine()
    _check(lib().egg_worker_engine_from_ctx(ctx._h, C.byref(e)))
    return e


class RunLog:
    """The reference's plain-text run log (header block + Step,RelTime,Loss,Updates,LR rows); no remote posting."""

    def __init__(self, path, cfg, num_gpus=1, vram_bytes_per_gpu=0):
        self._h = C.c_void_p()
        _check(lib().egg_log_open(path.encode(), C.byref(cfg), num_gpus, vram_bytes_per_gpu, C.byref(self._h)))

    def record(self, step, loss, updates, lr):
        _check(lib().egg_log_record(self._h, step, float(loss), int(updates), C.c_float(lr)))

    def close(self):
        if self._h:
            lib().egg_log_close(self._h)
            self._h = C.c_void_p()


class GruContext:
    """egg_gru_ctx: the recurrent model of full_trained_egg.c on one GPU (no CPU fallback)."""

    def __init__(self, gcfg, device=0):
        self.cfg = gcfg
        self._h = C.c_void_p()
        _check(lib().egg_gru_create(C.byref(gcfg), device, C.byref(self._h)))

    def close(self):
        if self._h:
            lib().egg_gru_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def upload_model(self, model):
        model = np.ascontiguousarray(model, np.int8)
        _check(lib().egg_gru_upload_model(self._h, _ptr(model), model.nbytes))

    def download_model(self):
        out = np.zeros(gru_model_bytes(self.cfg), np.int8)
        _check(lib().egg_gru_download_model(self._h, _ptr(out), out.nbytes))
        return out

    def upload_states(self, states):
        states = np.ascontiguousarray(states, np.int8)
        _check(lib().egg_gru_upload_states(self._h, _ptr(states), states.nbytes))

    def download_states(self):
        out = np.zeros(gru_state_bytes(self.cfg), np.int8)
        _check(lib().egg_gru_download_states(self._h, _ptr(out), out.nbytes))
        return out

    def set_dataset(self, tokens):
        tokens = np.ascontiguousarray(tokens, np.uint8)
        _check(lib().egg_gru_set_dataset(self._h, _ptr(tokens), tokens.nbytes))

    def generation(self, step_seed, start_idx, tokens, do_update=True):
        """Returns (losses[population], fitness[population/2])."""
        losses = np.zeros(self.cfg.population_size, np.int32)
        fit = np.zeros(self.cfg.population_size // 2, np.int32)
        _check(lib().egg_gru_generation(self._h, step_seed & 0xFFFFFFFF, start_idx, tokens, 1 if do_update else 0,
                                        _ptr(losses), _ptr(fit)))
        return losses, fit

    def launch_count(self):
        return lib().egg_gru_launch_count(self._h)
