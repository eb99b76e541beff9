// fns_compat.cu - fns::k::* with the reference's signatures (src/kernels.cuh:67-88) on top of the C ABI.
#include "../../include/fns_b200_compat.cuh"

#include <cstdio>
#include <cstdlib>
#include <mutex>

#include "../../include/fns_b200.h"

namespace {

constexpr int kCompatMaxDevices = 64;
constexpr int kCompatK = 64;  // the reference's kSampleMaxK (src/kernels.cu:598)

std::mutex g_lock;
fns_b200_sampler * g_handle[kCompatMaxDevices];
int g_vocab[kCompatMaxDevices];

[[noreturn]] void die(const char * what, const char * detail) {
    std::fprintf(stderr, "fns_b200 compat: %s: %s\n", what, detail ? detail : "");
    std::abort();
}

// One workspace per device, sized for one row (the reference samples one row per call), grown if a larger
// vocabulary shows up.
fns_b200_sampler * handle_for(int n) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kCompatMaxDevices) die("cudaGetDevice", "no device");
    std::lock_guard<std::mutex> hold(g_lock);
    if (g_handle[dev] && g_vocab[dev] >= n) return g_handle[dev];
    if (g_handle[dev]) fns_b200_destroy(g_handle[dev]);  // cudaFree waits for work in flight
    g_handle[dev] = nullptr;
    const int vocab = n < 262144 ? 262144 : n;
    if (fns_b200_create(dev, 1, vocab, kCompatK, 0, &g_handle[dev]) != FNS_B200_OK) die("fns_b200_create", "failed");
    g_vocab[dev] = vocab;
    return g_handle[dev];
}

void check(fns_b200_sampler * s, int rc, const char * what) {
    if (rc != FNS_B200_OK) die(what, s ? fns_b200_last_error(s) : "bad argument");
}

}  // namespace

namespace fns::k {

void argmax(const float * x, int n, int32_t * out, cudaStream_t st, const uint32_t * mask) {
    fns_b200_sampler * s = handle_for(n);
    fns_b200_params p{};
    p.temperature = 0.0f;  // greedy
    p.top_p = 1.0f;
    p.repetition = 1.0f;
    check(s, fns_b200_sample_one(s, x, FNS_B200_F32, n, mask, nullptr, 0, &p, out, st), "argmax");
}

void sample(const float * x, int n, const uint32_t * mask, int top_k, float top_p, float temperature, uint64_t seed,
            uint64_t counter, int32_t * out, cudaStream_t st) {
    fns_b200_sampler * s = handle_for(n);
    fns_b200_params p{};
    p.temperature = temperature;
    p.top_p = top_p;
    p.top_k = top_k;
    p.repetition = 1.0f;
    p.seed = seed;
    p.counter = counter;
    check(s, fns_b200_sample_one(s, x, FNS_B200_F32, n, mask, nullptr, 0, &p, out, st), "sample");
}

void presence_apply(float * x, const float * seen, int n, float penalty, cudaStream_t st) {
    check(nullptr, fns_b200_presence_apply(x, seen, n, penalty, st), "presence_apply");
}

void presence_mark(float * seen, const int32_t * token, cudaStream_t st) {
    check(nullptr, fns_b200_presence_mark(seen, token, st), "presence_mark");
}

void presence_apply_col(float * x, const float * seen, const int32_t * draft, int c, int n, float penalty,
                        cudaStream_t st) {
    check(nullptr, fns_b200_presence_apply_col(x, seen, draft, c, n, penalty, st), "presence_apply_col");
}

void presence_mark_n(float * seen, const int32_t * tokens, int n, cudaStream_t st) {
    check(nullptr, fns_b200_presence_mark_n(seen, tokens, n, st), "presence_mark_n");
}

void io_advance(int32_t * io, int pos, cudaStream_t st) {
    check(nullptr, fns_b200_io_advance(io, pos, st), "io_advance");
}

}  // namespace fns::k
