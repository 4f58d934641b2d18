// Runs the REFERENCE's own per-chunk fitness code: lines 635-687 of d-eggs/src/worker.cu
// (difference per pair, chunk-mean filter, mean-absolute-difference threshold, sign), which
// live inline in the worker's main().  oracle/Makefile cuts exactly those lines, unmodified,
// into oracle/_ref/worker_fitness_body.inc; this driver supplies the two names they read
// (`h_loss`, `count`) and prints the two they produce (`h_fit`, `sum_loss`).  The body is
// compiled four times, once per combination of the two compile-time switches of
// d-eggs/include/config.h:212-224.  TEST INFRASTRUCTURE ONLY.
//
//   ref_worker_fitness <mean_filter 0|1> <adaptive 0|1> < losses (text int32, one per token)
//   stdout: {"sum_loss": S, "fitness": [...]}
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <vector>

#include "config.h"

static void emit(const std::vector<int32_t> &h_fit, int64_t sum_loss) {
    printf("{\"sum_loss\": %lld, \"fitness\": [", (long long)sum_loss);
    for (size_t i = 0; i < h_fit.size(); i++) printf("%s%d", i ? ", " : "", (int)h_fit[i]);
    printf("]}\n");
}

#undef CHUNK_MEAN_FILTER
#undef USE_ADAPTIVE_THRESHOLD
#define CHUNK_MEAN_FILTER 1
#define USE_ADAPTIVE_THRESHOLD 1
static void body_11(std::vector<int32_t> &h_loss, int count) {
#include "worker_fitness_body.inc"
    emit(h_fit, sum_loss);
}
#undef CHUNK_MEAN_FILTER
#undef USE_ADAPTIVE_THRESHOLD
#define CHUNK_MEAN_FILTER 0
#define USE_ADAPTIVE_THRESHOLD 1
static void body_01(std::vector<int32_t> &h_loss, int count) {
#include "worker_fitness_body.inc"
    emit(h_fit, sum_loss);
}
#undef CHUNK_MEAN_FILTER
#undef USE_ADAPTIVE_THRESHOLD
#define CHUNK_MEAN_FILTER 1
#define USE_ADAPTIVE_THRESHOLD 0
static void body_10(std::vector<int32_t> &h_loss, int count) {
#include "worker_fitness_body.inc"
    emit(h_fit, sum_loss);
}
#undef CHUNK_MEAN_FILTER
#undef USE_ADAPTIVE_THRESHOLD
#define CHUNK_MEAN_FILTER 0
#define USE_ADAPTIVE_THRESHOLD 0
static void body_00(std::vector<int32_t> &h_loss, int count) {
#include "worker_fitness_body.inc"
    emit(h_fit, sum_loss);
}

int main(int argc, char **argv) {
    if (argc < 3) { fprintf(stderr, "usage: ref_worker_fitness <mean_filter> <adaptive> < losses\n"); return 2; }
    const int mf = atoi(argv[1]), ad = atoi(argv[2]);
    std::vector<int32_t> h_loss;
    long long v;
    while (scanf("%lld", &v) == 1) h_loss.push_back((int32_t)v);
    const int count = (int)h_loss.size();
    if (count < 2 || (count & 1)) { fprintf(stderr, "need an even number of losses\n"); return 2; }
    if (mf && ad) body_11(h_loss, count);
    else if (!mf && ad) body_01(h_loss, count);
    else if (mf && !ad) body_10(h_loss, count);
    else body_00(h_loss, count);
    return 0;
}
