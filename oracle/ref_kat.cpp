// Known-answer generator: compiles the REFERENCE's own host-callable headers
// (d-eggs/include/utils/egg_math.h, ternary_pack.h) and prints their outputs as
// JSON.  Built into oracle/_ref/ref_kat by oracle/Makefile; its output is
// committed as tests/golden/rng_kat.json (see tests/golden/make_golden.py).
// Usage: ref_kat            (DEVICE_MASK / HOST_MASK come from -D, default 15)
#include <cstdio>
#include <cstdint>
#include <vector>
#include "utils/egg_math.h"
#include "utils/ternary_pack.h"
#include "protocol.h"

int main() {
    printf("{\n \"device_mask\": %d, \"host_mask\": %d,\n", DEVICE_MASK, HOST_MASK);
    const uint32_t seeds[] = {0u, 1u, 42u, 0xFFFFFFFFu, 12648430u, 0x00C0FFEEu, 2u};
    const uint32_t idxs[] = {0u, 1u, 511u, 0xFFFFFFFFu, 4095u};
    printf(" \"hash_rng\": [");
    bool first = true;
    for (uint32_t s : seeds) for (uint32_t i : idxs) {
        printf("%s[%u, %u, %u]", first ? "" : ", ", s, i, hash_rng(s, i)); first = false;
    }
    printf("],\n \"noise\": [");
    first = true;
    for (uint32_t s : seeds) {
        printf("%s{\"seed\": %u, \"values\": [", first ? "" : ", ", s); first = false;
        for (uint32_t i = 0; i < 64; i++) printf("%s%d", i ? ", " : "", (int)noise_from_hash(s, i));
        printf("]}");
    }
    printf("],\n \"gen_noise_host\": {\"state\": 42, \"values\": [");
    uint32_t st = 42;
    for (int i = 0; i < 64; i++) printf("%s%d", i ? ", " : "", (int)gen_noise_host(&st));
    printf("]},\n \"ternary\": [");
    // the two round-trip cases of d-eggs/test_ternary.cpp plus an LCG stream
    std::vector<std::vector<int32_t>> cases = {
        {-1, 0, 1, -1, 0, 1, 1, 0, -1, 0}, {-1, 0, 1, -1, 0, 1, 1}, {}, {1}, {-1, -1, -1, -1, -1}};
    std::vector<int32_t> lcg; uint32_t x = 12345;
    for (int i = 0; i < 103; i++) { x = x * 1664525u + 1013904223u; lcg.push_back((int)((x >> 16) % 3) - 1); }
    cases.push_back(lcg);
    first = true;
    for (auto &c : cases) {
        std::vector<uint8_t> packed(ternary_pack_estimate_size(c.size()) + 1, 0);
        ternary_pack(c.data(), c.size(), packed.data());
        printf("%s{\"values\": [", first ? "" : ", "); first = false;
        for (size_t i = 0; i < c.size(); i++) printf("%s%d", i ? ", " : "", c[i]);
        printf("], \"packed\": [");
        for (size_t i = 0; i < ternary_pack_estimate_size(c.size()); i++) printf("%s%u", i ? ", " : "", packed[i]);
        printf("]}");
    }
    printf("],\n \"wire\": [");
    // the three message kinds of d-eggs/include/protocol.h, serialised by the reference's own helpers
    auto hex = [](const uint8_t *b, int n) { for (int i = 0; i < n; i++) printf("%02x", b[i]); };
    {
        uint8_t buf[64];
        EggJobRequest rq = {0x1122334455667788ull, 930, 0xFFFFFFFFFFFFFFFFull};
        egg_write_header(buf, OP_JOB_REQUEST, 24); egg_serialize_job_request(buf + 10, &rq);
        printf("{\"opcode\": 0, \"seed\": %llu, \"last_step\": %llu, \"data_position\": %llu, \"payload_size\": 0, \"updates_count\": 0, \"sum_loss\": 0, \"hex\": \"",
               (unsigned long long)rq.seed, (unsigned long long)rq.last_step, (unsigned long long)rq.data_position);
        hex(buf, 34); printf("\"}, ");
        EggJobResponseHeader rs = {42, 7, 123456789012ull, 26215};
        egg_write_header(buf, OP_JOB_RESPONSE, 28 + rs.model_size); egg_serialize_job_response_header(buf + 10, &rs);
        printf("{\"opcode\": 2, \"seed\": 42, \"last_step\": 7, \"data_position\": 123456789012, \"payload_size\": 26215, \"updates_count\": 0, \"sum_loss\": 0, \"hex\": \"");
        hex(buf, 38); printf("\"}, ");
        EggResultHeader rr = {0xC0FFEE, 15470, 4096, 591871, (uint64_t)(int64_t)-123456789, 3277};
        egg_write_header(buf, OP_RESULT, 44 + rr.result_size); egg_serialize_result_header(buf + 10, &rr);
        printf("{\"opcode\": 1, \"seed\": %u, \"last_step\": 15470, \"data_position\": 4096, \"payload_size\": 3277, \"updates_count\": 591871, \"sum_loss\": -123456789, \"hex\": \"", 0xC0FFEE);
        hex(buf, 54); printf("\"}");
    }
    printf("]\n}\n");
    return 0;
}
