// Host side of the d-eggs worker and the run log (no CUDA in this file).
//
// * egg_log_*: the reference's CSV run log (egg_disk_log.h:93-139 header block and column line, :206-224 one row per
//   step) without its remote posting: nothing here opens a network connection.
// * egg_worker_run: the worker loop of d-eggs/src/worker.cu:390-717 -- JOB_REQUEST, then either an update (packed
//   fitness of the whole population -> optimiser step -> seed chain), a wait, or a chunk (evaluate CHUNK_SIZE members,
//   per-chunk fitness filter, ternary pack, RESULT) -- speaking d-eggs/include/protocol.h to an unmodified
//   coordinator.  The GPU work sits behind a small table of callbacks (egg_worker_engine): egg_worker_engine_from_ctx
//   binds it to an egg_ctx of this library; tests bind host-side fakes to exercise the control flow and the fault cases
//   (a worker that stops answering, stale and duplicate results, a late joiner) without a GPU.
#include "../../include/egg_b200.h"

#include <arpa/inet.h>
#include <errno.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <poll.h>
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <sys/socket.h>
#include <time.h>
#include <unistd.h>

#include <string>
#include <vector>

namespace egg {
void set_error(const char *fmt, ...);
}
using egg::set_error;

// ---------------------------------------------------------------- run log

struct egg_log {
    std::string path;
    struct timespec start;
};

extern "C" int egg_log_open(const char *path, const egg_config *c, int num_gpus, uint64_t vram_bytes_per_gpu, egg_log **out) {
    if (!path || !c || !out) { set_error("null argument"); return EGG_E_INVALID; }
    *out = nullptr;
    FILE *f = fopen(path, "a");
    if (!f) { set_error("cannot open %s: %s", path, strerror(errno)); return EGG_E_INVALID; }
    fseek(f, 0, SEEK_END);
    if (ftell(f) > 0) fprintf(f, "\n");                 // a blank line between runs that share a file
    time_t raw = time(nullptr);
    char when[64];
    strftime(when, sizeof(when), "%Y-%m-%dT%H:%M:%S", localtime(&raw));
    // the header block and the column line of egg_disk_log.h:111-139, field for field
    fprintf(f, "=== Training Run ===\n");
    fprintf(f, "Run Start:       %s\n", when);
    fprintf(f, "Hardware:        %d GPUs, %.2f MB VRAM/GPU\n", num_gpus, (double)vram_bytes_per_gpu / (1024.0 * 1024.0));
    fprintf(f, "Model Config:    Hidden=%d, Head=%d, Layers=%d, SeqLen=%d\n", c->hidden_dim, c->head_dim, c->n_layers, c->seq_len);
    fprintf(f, "                 Vocab=%d, Heads=%d, PopSize=%d, SoftmaxScaleBit=%d\n", c->vocab_size, c->hidden_dim / c->head_dim,
            c->population_size, c->softmax_scale_bit);
    fprintf(f, "Noise Config:    HostGaussian=%d, DeviceGaussian=%d, HostMask=%d, DeviceMask=%d\n", 0, c->device_gaussian, c->host_mask,
            c->device_mask);
    fprintf(f, "Quant Config:    FixedPoint=%d, SigmaShift=%d, SigmaShiftVec=%d\n", c->fixed_point, c->sigma_shift, c->sigma_shift_vector);
    fprintf(f, "Shift Config:    Attn=%d, QKV=%d, Out=%d, Logit=%d, MLP_Up=%d, MLP_Dn=%d\n", c->shift_attn, 6, c->shift_out, c->shift_logit,
            c->shift_mlp_up, c->shift_mlp_down);
    fprintf(f, "Optimizer:       Adam(B1=%.3f, B2=%.3f, Eps=%.1e, WD=%.4f)\n", c->adam_beta1, c->adam_beta2, c->adam_eps, c->adam_weight_decay);
    if (c->use_muon) fprintf(f, "                 Muon(Mom=%.3f, Scale=%.3f)\n", c->muon_momentum, c->muon_lr_scale);
    fprintf(f, "Misc:            SoftmaxExpScale=%.2f\n", c->softmax_exp_scale);
    fprintf(f, "----------------------------------------------------------------\n");
    fprintf(f, "Step,RelTime,Loss,Updates,LR\n");
    fclose(f);
    egg_log *l = new egg_log();
    l->path = path;
    clock_gettime(CLOCK_MONOTONIC, &l->start);
    *out = l;
    return EGG_OK;
}

extern "C" int egg_log_record(egg_log *l, int64_t step, double loss, uint64_t updates, float lr) {
    if (!l) { set_error("null log"); return EGG_E_INVALID; }
    struct timespec now;
    clock_gettime(CLOCK_MONOTONIC, &now);
    const double rel = (double)(now.tv_sec - l->start.tv_sec) + (double)(now.tv_nsec - l->start.tv_nsec) / 1e9;
    FILE *f = fopen(l->path.c_str(), "a");
    if (!f) { set_error("cannot open %s: %s", l->path.c_str(), strerror(errno)); return EGG_E_INVALID; }
    fprintf(f, "%ld,%.4f,%.4f,%llu,%.6f\n", (long)step, rel, loss, (unsigned long long)updates, lr);   // egg_disk_log.h:222
    fclose(f);
    return EGG_OK;
}

extern "C" void egg_log_close(egg_log *l) { delete l; }

// ---------------------------------------------------------------- worker

extern "C" float egg_learning_rate(int64_t step) {        // d-eggs/include/utils/training.h:5-9
    if (step < 100) return 0.5f;
    if (step < 200) return 0.25f;
    return 0.125f;
}

namespace {

bool send_all(int fd, const void *buf, size_t n) {
    const uint8_t *p = static_cast<const uint8_t *>(buf);
    while (n) {
        ssize_t w = send(fd, p, n, MSG_NOSIGNAL);
        if (w <= 0) { if (w < 0 && errno == EINTR) continue; return false; }
        p += w; n -= (size_t)w;
    }
    return true;
}

// false on a closed connection, an error or when nothing arrives for timeout_ms (a coordinator that went away)
bool recv_all(int fd, void *buf, size_t n, int timeout_ms) {
    uint8_t *p = static_cast<uint8_t *>(buf);
    while (n) {
        struct pollfd pf = {fd, POLLIN, 0};
        int pr = poll(&pf, 1, timeout_ms);
        if (pr == 0) return false;
        if (pr < 0) { if (errno == EINTR) continue; return false; }
        ssize_t r = recv(fd, p, n, 0);
        if (r <= 0) { if (r < 0 && errno == EINTR) continue; return false; }
        p += r; n -= (size_t)r;
    }
    return true;
}

bool send_msg(int fd, const egg_wire_msg &m, const void *payload, uint64_t *bytes_out) {
    uint8_t fixed[64];
    const int nfix = egg_wire_encode(&m, fixed, (int)sizeof(fixed));
    if (nfix < 0) return false;
    if (!send_all(fd, fixed, (size_t)nfix)) return false;
    if (m.payload_size && !send_all(fd, payload, m.payload_size)) return false;
    if (bytes_out) *bytes_out += (uint64_t)nfix + m.payload_size;
    return true;
}

}  // namespace

extern "C" void egg_worker_options_defaults(egg_worker_options *o) {
    memset(o, 0, sizeof(*o));
    snprintf(o->host, sizeof(o->host), "127.0.0.1");
    o->port = 12345;                     // coordinator.cpp:26
    o->initial_seed = 42;                // worker.cu:386
    o->wait_sleep_ms = 100;              // worker.cu:552
    o->recv_timeout_ms = 30000;
    o->generate_every = 5;               // worker.cu:564
    o->mean_filter = 1; o->mean_exponent = 1.2; o->adaptive_threshold = 1; o->threshold_alpha = 0.1;   // config.h:212-224
    o->stop_at_step = -1; o->max_requests = -1;
}

extern "C" int egg_worker_run(const egg_worker_options *o, const egg_worker_engine *eng, egg_worker_stats *stats) {
    if (!o || !eng || !eng->eval_chunk || !eng->apply_update) { set_error("worker needs options and an engine with eval_chunk and apply_update"); return EGG_E_INVALID; }
    if (o->chunk_size < 2 || (o->chunk_size & 1) || o->population_size < o->chunk_size || o->population_size % o->chunk_size) {
        set_error("population %d must be a multiple of the even chunk size %d", o->population_size, o->chunk_size);
        return EGG_E_INVALID;
    }
    egg_worker_stats st;
    memset(&st, 0, sizeof(st));
    auto finish = [&](int rc) { if (stats) *stats = st; return rc; };

    int fd = socket(AF_INET, SOCK_STREAM, 0);
    if (fd < 0) { set_error("socket: %s", strerror(errno)); return finish(EGG_E_STATE); }
    int one = 1;
    setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
    struct sockaddr_in addr;
    memset(&addr, 0, sizeof(addr));
    addr.sin_family = AF_INET;
    addr.sin_port = htons((uint16_t)o->port);
    if (inet_pton(AF_INET, o->host, &addr.sin_addr) != 1) { close(fd); set_error("bad coordinator address %s", o->host); return finish(EGG_E_INVALID); }
    if (connect(fd, (struct sockaddr *)&addr, sizeof(addr)) < 0) { close(fd); set_error("cannot connect to %s:%d: %s", o->host, o->port, strerror(errno)); return finish(EGG_E_STATE); }

    uint64_t step = 0, seed = o->initial_seed, last_updates = 0;
    const int pairs_all = o->population_size / 2;
    std::vector<int32_t> fit_all((size_t)pairs_all), losses((size_t)o->chunk_size), fit_chunk((size_t)o->chunk_size / 2);
    std::vector<uint8_t> payload, packed((size_t)egg_ternary_packed_size(o->chunk_size / 2));
    int rc = EGG_OK;
    while (true) {
        if (o->stop_at_step >= 0 && (int64_t)step >= o->stop_at_step) break;
        if (o->max_requests >= 0 && (int64_t)st.requests >= o->max_requests) break;
        if (o->stop_flag && *o->stop_flag) break;
        // JOB_REQUEST (worker.cu:392-399)
        egg_wire_msg req;
        memset(&req, 0, sizeof(req));
        req.opcode = EGG_OP_JOB_REQUEST; req.seed = seed; req.last_step = step;
        if (!send_msg(fd, req, nullptr, &st.bytes_sent)) { set_error("coordinator connection lost while sending a request"); rc = EGG_E_STATE; break; }
        st.requests++;
        uint8_t hdr[EGG_WIRE_HEADER_BYTES];
        const int hdr_len = EGG_WIRE_HEADER_BYTES;
        if (!recv_all(fd, hdr, (size_t)hdr_len, o->recv_timeout_ms)) { set_error("coordinator stopped answering"); rc = EGG_E_STATE; break; }
        int opcode = 0; uint32_t plen = 0;
        if (egg_wire_decode_header(hdr, &opcode, &plen)) { set_error("bad packet header from the coordinator"); rc = EGG_E_INVALID; break; }
        payload.resize(plen);
        if (plen && !recv_all(fd, payload.data(), plen, o->recv_timeout_ms)) { set_error("coordinator stopped answering inside a packet"); rc = EGG_E_STATE; break; }
        st.bytes_received += (uint64_t)hdr_len + plen;
        if (opcode != EGG_OP_JOB_RESPONSE) continue;                  // worker.cu:409: anything else is ignored
        egg_wire_msg resp;
        if (egg_wire_decode_body(opcode, payload.data(), (int)plen, &resp)) { set_error("short JOB_RESPONSE"); rc = EGG_E_INVALID; break; }

        if (resp.payload_size > 0) {
            // update: packed fitness of the whole population for the worker's step (worker.cu:416-547)
            const int64_t need = egg_ternary_packed_size(pairs_all);
            if ((int64_t)resp.payload_size < need || (int64_t)plen < 28 + need) { set_error("update carries %u fitness bytes, need %lld", resp.payload_size, (long long)need); rc = EGG_E_INVALID; break; }
            egg_ternary_unpack(payload.data() + 28, pairs_all, fit_all.data());
            const float lr = egg_learning_rate((int64_t)step);
            uint64_t upd = 0;
            if ((rc = eng->apply_update(eng->self, fit_all.data(), pairs_all, (uint32_t)seed, lr, lr * 0.1f, &upd))) break;
            last_updates = upd;
            st.updates_applied++;
            step = resp.last_step;                                   // worker.cu:541
            seed = egg_next_seed((uint32_t)seed, (uint32_t)step);    // worker.cu:542
            continue;
        }
        if (resp.data_position == UINT64_MAX) {                      // nothing to do right now (worker.cu:550-554)
            st.waits++;
            if (o->wait_sleep_ms > 0) { struct timespec ts = {o->wait_sleep_ms / 1000, (long)(o->wait_sleep_ms % 1000) * 1000000L}; nanosleep(&ts, nullptr); }
            continue;
        }
        // a chunk (worker.cu:557-713)
        const int pop_offset = (int)resp.data_position;
        const int chunk_idx = pop_offset / o->chunk_size;
        if (pop_offset < 0 || pop_offset + o->chunk_size > o->population_size) { set_error("chunk at %d outside the population", pop_offset); rc = EGG_E_INVALID; break; }
        if (eng->generate && o->generate_every > 0 && chunk_idx == 0 && step % (uint64_t)o->generate_every == 0) {
            char text[1024];
            int n = eng->generate(eng->self, (int64_t)step, (uint32_t)seed + 999u, text, (int)sizeof(text));   // worker.cu:564-613
            if (n > 0) {
                egg_wire_msg lg;
                memset(&lg, 0, sizeof(lg));
                lg.opcode = EGG_OP_LOG_MESSAGE; lg.payload_size = (uint32_t)n;
                if (!send_msg(fd, lg, text, &st.bytes_sent)) { set_error("coordinator connection lost while sending a log message"); rc = EGG_E_STATE; break; }
            }
        }
        if ((rc = eng->eval_chunk(eng->self, (uint32_t)seed, (int64_t)step, pop_offset, o->chunk_size, losses.data()))) break;
        int64_t sum_loss = 0;
        egg_deggs_chunk_fitness(losses.data(), o->chunk_size, o->mean_filter, o->mean_exponent, o->adaptive_threshold, o->threshold_alpha,
                                fit_chunk.data(), &sum_loss);
        egg_ternary_pack(fit_chunk.data(), o->chunk_size / 2, packed.data());
        egg_wire_msg res;
        memset(&res, 0, sizeof(res));
        res.opcode = EGG_OP_RESULT; res.seed = seed; res.last_step = step; res.data_position = resp.data_position;
        res.updates_count = last_updates; res.sum_loss = sum_loss; res.payload_size = (uint32_t)packed.size();
        last_updates = 0;                                            // worker.cu:701
        if (o->before_result && o->before_result(o->hook_self, (int64_t)step, chunk_idx)) { st.results_dropped++; continue; }
        if (!send_msg(fd, res, packed.data(), &st.bytes_sent)) { set_error("coordinator connection lost while sending a result"); rc = EGG_E_STATE; break; }
        st.chunks_done++;
    }
    close(fd);
    st.final_step = step; st.final_seed = seed;
    return finish(rc);
}

// ---- the engine backed by an egg_ctx ----
namespace {
int ctx_eval_chunk(void *self, uint32_t seed, int64_t step, int pop_offset, int count, int32_t *losses) {
    egg_ctx *c = static_cast<egg_ctx *>(self);
    egg_config cfg;
    int rc = egg_get_config(c, &cfg);
    if (rc) return rc;
    // train_sequence_kernel<<<count>>>(..., current_step*SEQ_LEN, ..., current_seed, global_pop_offset, ...), worker.cu:626-629
    if ((rc = egg_eval_chunk(c, seed, step * cfg.seq_len, pop_offset, count))) return rc;
    // d-eggs writes the losses chunk-relative (kernels.cu:297), the mgpu trainer by global member index (mgpu.cu:1028)
    return egg_read_losses(c, losses, cfg.chunk_relative_loss ? 0 : pop_offset, count);
}

int ctx_apply_update(void *self, const int32_t *fitness, int pairs, uint32_t seed, float lr, float lr_bias, uint64_t *updates) {
    egg_ctx *c = static_cast<egg_ctx *>(self);
    (void)lr_bias;                       // emb_bias takes 0.1 * lr inside the library, as worker.cu:428 passes it
    int rc = egg_write_fitness(c, fitness, 0, pairs);
    if (rc) return rc;
    return egg_apply_update(c, seed, lr, updates);
}
}  // namespace

extern "C" int egg_worker_engine_from_ctx(egg_ctx *ctx, egg_worker_engine *out) {
    if (!ctx || !out) { set_error("null argument"); return EGG_E_INVALID; }
    memset(out, 0, sizeof(*out));
    out->self = ctx;
    out->eval_chunk = ctx_eval_chunk;
    out->apply_update = ctx_apply_update;
    out->generate = nullptr;
    return EGG_OK;
}
