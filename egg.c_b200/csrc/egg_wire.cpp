// Host-side pieces of the d-eggs worker boundary: wire messages, the 5-trits-per-byte fitness
// codec, the per-chunk host fitness filter and the seed chain.  Plain C++ (no CUDA): these run on
// the worker's host thread between kernel launches in the reference too.
#include <math.h>
#include <stdlib.h>
#include <string.h>

#include <vector>

#include "../../include/egg_b200.h"

namespace {

// big-endian field writers/readers (the reference converts with htonl/htonll, protocol.h:21-33)
void put_be(uint8_t *p, uint64_t v, int nbytes) {
    for (int i = nbytes - 1; i >= 0; i--) { p[i] = (uint8_t)(v & 0xFF); v >>= 8; }
}
uint64_t get_be(const uint8_t *p, int nbytes) {
    uint64_t v = 0;
    for (int i = 0; i < nbytes; i++) v = (v << 8) | p[i];
    return v;
}
const uint32_t kMagic = 0x4A4F4253u;   // "JOBS", protocol.h:8

}  // namespace

// fixed body size of a message kind: JOB_REQUEST 24, RESULT 44, JOB_RESPONSE 28 (protocol.h:61-160)
extern "C" int egg_wire_fixed_bytes(int opcode) {
    switch (opcode) {
        case EGG_OP_JOB_REQUEST: return 24;
        case EGG_OP_RESULT: return 44;
        case EGG_OP_JOB_RESPONSE: return 28;
        case EGG_OP_LOG_MESSAGE: return 0;
    }
    return -1;
}

// Writes the 10-byte header followed by the fixed body; the variable payload (packed fitness, log text)
// follows on the wire and is counted in the header's length through msg->payload_size.
extern "C" int egg_wire_encode(const egg_wire_msg *m, uint8_t *out, int cap) {
    if (!m || !out) return EGG_E_INVALID;
    const int body = egg_wire_fixed_bytes(m->opcode);
    if (body < 0 || cap < EGG_WIRE_HEADER_BYTES + body) return EGG_E_INVALID;
    put_be(out, kMagic, 4);
    out[4] = 1;                                  // EGG_PROTO_VERSION
    out[5] = (uint8_t)m->opcode;
    put_be(out + 6, (uint64_t)body + m->payload_size, 4);
    uint8_t *b = out + EGG_WIRE_HEADER_BYTES;
    if (body >= 24) { put_be(b, m->seed, 8); put_be(b + 8, m->last_step, 8); put_be(b + 16, m->data_position, 8); }
    if (m->opcode == EGG_OP_JOB_RESPONSE) put_be(b + 24, m->payload_size, 4);
    if (m->opcode == EGG_OP_RESULT) {
        put_be(b + 24, m->updates_count, 8);
        put_be(b + 32, (uint64_t)m->sum_loss, 8);
        put_be(b + 40, m->payload_size, 4);
    }
    return EGG_WIRE_HEADER_BYTES + body;
}

// -1: bad magic, -2: bad version (the reference's egg_parse_header return codes, protocol.h:46-56)
extern "C" int egg_wire_decode_header(const uint8_t *buf10, int *opcode, uint32_t *total_len) {
    if (!buf10 || !opcode || !total_len) return EGG_E_INVALID;
    if ((uint32_t)get_be(buf10, 4) != kMagic) return -1;
    if (buf10[4] != 1) return -2;
    *opcode = buf10[5];
    *total_len = (uint32_t)get_be(buf10 + 6, 4);
    return 0;
}

extern "C" int egg_wire_decode_body(int opcode, const uint8_t *body, int len, egg_wire_msg *m) {
    const int need = egg_wire_fixed_bytes(opcode);
    if (!body || !m || need < 0 || len < need) return EGG_E_INVALID;
    memset(m, 0, sizeof(*m));
    m->opcode = opcode;
    if (need >= 24) { m->seed = get_be(body, 8); m->last_step = get_be(body + 8, 8); m->data_position = get_be(body + 16, 8); }
    if (opcode == EGG_OP_JOB_RESPONSE) m->payload_size = (uint32_t)get_be(body + 24, 4);
    if (opcode == EGG_OP_RESULT) {
        m->updates_count = get_be(body + 24, 8);
        m->sum_loss = (int64_t)get_be(body + 32, 8);
        m->payload_size = (uint32_t)get_be(body + 40, 4);
    }
    return 0;
}

// ---- fitness codec: base 3, five values per byte, digit = (v+3)%3, least significant first (ternary_pack.h:12-87)
extern "C" int64_t egg_ternary_packed_size(int64_t count) { return (count + 4) / 5; }

extern "C" void egg_ternary_pack(const int32_t *values, int64_t count, uint8_t *out) {
    static const int pow3[5] = {1, 3, 9, 27, 81};
    for (int64_t base = 0, o = 0; base < count; base += 5, o++) {
        int acc = 0;
        const int n = (int)((count - base) < 5 ? (count - base) : 5);
        for (int j = 0; j < n; j++) acc += ((values[base + j] + 3) % 3) * pow3[j];
        out[o] = (uint8_t)acc;
    }
}

extern "C" void egg_ternary_unpack(const uint8_t *in, int64_t count, int32_t *values) {
    for (int64_t base = 0, o = 0; base < count; base += 5, o++) {
        int acc = in[o];
        const int n = (int)((count - base) < 5 ? (count - base) : 5);
        for (int j = 0; j < n; j++) { int d = acc % 3; acc /= 3; values[base + j] = d == 2 ? -1 : d; }
    }
}

// ---- per-chunk host fitness of the d-eggs worker (worker.cu:635-687): loss differences, the chunk-mean
// filter diff += (int)(sgn * pow(|mean|, exponent)), then the MAD threshold |diff| < alpha*MAD -> 0.
extern "C" int egg_deggs_chunk_fitness(const int32_t *losses, int count, int mean_filter, double exponent, int adaptive_threshold,
                                       double alpha, int32_t *fitness, int64_t *sum_loss) {
    if (!losses || !fitness || count < 2 || (count & 1)) return EGG_E_INVALID;
    const int n = count / 2;
    std::vector<int32_t> diffs((size_t)n);
    int64_t sum = 0;
    double sum_diff = 0.0;
    for (int i = 0; i < n; i++) {
        const int32_t p = losses[2 * i], q = losses[2 * i + 1];
        sum += (int64_t)p + q;
        diffs[i] = q - p;
        sum_diff += diffs[i];
    }
    if (mean_filter) {
        double mean_diff = sum_diff / n;
        if (mean_diff != 0.0) mean_diff = (mean_diff > 0 ? 1.0 : -1.0) * pow(fabs(mean_diff), exponent);
        const int32_t shift = (int32_t)mean_diff;
        for (int i = 0; i < n; i++) diffs[i] += shift;
    }
    if (adaptive_threshold) {
        double sum_abs = 0.0;
        for (int i = 0; i < n; i++) sum_abs += fabs((double)diffs[i]);
        const double threshold = (sum_abs / n) * alpha;
        for (int i = 0; i < n; i++) fitness[i] = fabs((double)diffs[i]) < threshold ? 0 : (diffs[i] > 0 ? 1 : -1);
    } else {
        for (int i = 0; i < n; i++) fitness[i] = diffs[i] > 0 ? 1 : (diffs[i] < 0 ? -1 : 0);
    }
    if (sum_loss) *sum_loss = sum;
    return EGG_OK;
}

// seed chain of worker and coordinator: seed' = hash_rng((u32)seed, step) (worker.cu:542, coordinator.cpp:406)
extern "C" uint32_t egg_next_seed(uint32_t seed, uint64_t step) {
    uint32_t x = seed + (uint32_t)step * 0x9e3779b9u;
    x ^= x >> 16; x *= 0x85ebca6bu;
    x ^= x >> 13; x *= 0xc2b2ae35u;
    x ^= x >> 16;
    return x;
}
