// ref_harness.cu - C entry points around the reference's own sampler functions (fns::k::*, declared in
// the reference's src/kernels.cuh:67-88), so that tests and the benchmark can drive the UNMODIFIED
// reference kernels, recompiled for sm_100a, through ctypes.
//
// TEST INFRASTRUCTURE ONLY: the checker and the "reference on the same GPU" timing arm.  The shipped
// library never links or loads this.  The reference sources are compiled where they lie (see Makefile);
// nothing of them is copied here.  All pointers are device pointers unless a name ends in _host.
#include "kernels.cuh"

#include <cuda_runtime.h>

#include <cstdint>

extern "C" {

void fns_ref_sample(const float * x, int n, const uint32_t * mask, int top_k, float top_p, float temperature,
                    uint64_t seed, uint64_t counter, int32_t * out, void * stream) {
    fns::k::sample(x, n, mask, top_k, top_p, temperature, seed, counter, out, (cudaStream_t) stream);
}

void fns_ref_argmax(const float * x, int n, int32_t * out, void * stream, const uint32_t * mask) {
    fns::k::argmax(x, n, out, (cudaStream_t) stream, mask);
}

void fns_ref_presence_apply(float * x, const float * seen, int n, float penalty, void * stream) {
    fns::k::presence_apply(x, seen, n, penalty, (cudaStream_t) stream);
}

void fns_ref_presence_mark(float * seen, const int32_t * token, void * stream) {
    fns::k::presence_mark(seen, token, (cudaStream_t) stream);
}

void fns_ref_presence_apply_col(float * x, const float * seen, const int32_t * draft, int c, int n, float penalty,
                                void * stream) {
    fns::k::presence_apply_col(x, seen, draft, c, n, penalty, (cudaStream_t) stream);
}

void fns_ref_presence_mark_n(float * seen, const int32_t * tokens, int n, void * stream) {
    fns::k::presence_mark_n(seen, tokens, n, (cudaStream_t) stream);
}

void fns_ref_io_advance(int32_t * io, int pos, void * stream) { fns::k::io_advance(io, pos, (cudaStream_t) stream); }

// Rows one after another on one stream: the reference is one row per call and not re-entrant (its
// candidates go through file-scope device arrays, src/kernels.cu:601-602).  Per-row scalars are host arrays;
// temperature <= 0 takes the argmax entry point as Engine::pick_async does (src/engine.cu:841-842).
void fns_ref_sample_rows(const float * x, int64_t row_stride, int n, int rows, const uint32_t * masks,
                         int64_t mask_stride, const int32_t * top_k_host, const float * top_p_host,
                         const float * temperature_host, const uint64_t * seed_host, const uint64_t * counter_host,
                         int32_t * out, void * stream) {
    for (int r = 0; r < rows; ++r) {
        const uint32_t * m = masks ? masks + r * mask_stride : nullptr;
        if (temperature_host[r] <= 0.0f)
            fns::k::argmax(x + r * row_stride, n, out + r, (cudaStream_t) stream, m);
        else
            fns::k::sample(x + r * row_stride, n, m, top_k_host[r], top_p_host[r], temperature_host[r], seed_host[r],
                           counter_host[r], out + r, (cudaStream_t) stream);
    }
}

// The same draw repeated with counters counter0 .. counter0 + draws - 1 into out[draws]
// (the loop of tests/sample_check.cu:35).
void fns_ref_sample_counters(const float * x, int n, const uint32_t * mask, int top_k, float top_p, float temperature,
                             uint64_t seed, uint64_t counter0, int draws, int32_t * out, void * stream) {
    for (int i = 0; i < draws; ++i)
        fns::k::sample(x, n, mask, top_k, top_p, temperature, seed, counter0 + (uint64_t) i, out + i,
                       (cudaStream_t) stream);
}

}  // extern "C"
