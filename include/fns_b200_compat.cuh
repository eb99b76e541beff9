// fns_b200_compat.cuh - the reference's sampler entry points, same namespace, names and signatures
// (NomenAK/FlintNSteel src/kernels.cuh:67-88), implemented by libfns_b200.so.
//
// An engine that calls fns::k::argmax / sample / presence_* / io_advance (src/engine.cu:368,754-756,798,807,
// 839-843,865; src/exl3/exl3_engine.cu:675,688,701-708,730) links this library in place of those seven
// definitions in src/kernels.cu and needs no source change.  Differences a caller can observe:
//   * candidates live in a per-device workspace created on the first call (the only allocation, and it
//     happens outside any stream capture if the first call does), not in file-scope device arrays;
//   * errors print to stderr and abort, as the reference's FNS_CHECK does (src/kernels.cu:9-16).
#pragma once

#include <cuda_runtime.h>

#include <cstdint>

namespace fns::k {

// *out = first allowed finite element of x in the order (value descending, index ascending).  kernels.cuh:69
void argmax(const float * x, int n, int32_t * out, cudaStream_t st, const uint32_t * mask = nullptr);

// top-k / top-p / temperature / Philox (seed, counter); top_k <= 0 or > 64: 64; temperature <= 0: argmax;
// *out = -1 if no token is allowed.  kernels.cuh:74-75
void sample(const float * x, int n, const uint32_t * mask, int top_k, float top_p, float temperature, uint64_t seed,
            uint64_t counter, int32_t * out, cudaStream_t st);

void presence_apply(float * x, const float * seen, int n, float penalty, cudaStream_t st);           // kernels.cuh:79
void presence_mark(float * seen, const int32_t * token, cudaStream_t st);                            // kernels.cuh:80
void presence_apply_col(float * x, const float * seen, const int32_t * draft, int c, int n, float penalty,
                        cudaStream_t st);                                                            // kernels.cuh:83-84
void presence_mark_n(float * seen, const int32_t * tokens, int n, cudaStream_t st);                  // kernels.cuh:85
void io_advance(int32_t * io, int pos, cudaStream_t st);                                             // kernels.cuh:88

}  // namespace fns::k
