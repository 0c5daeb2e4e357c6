// A row-major activation that is either stored in the activation type or still split into the
// float32 partial sums [parts, tokens, row_stride] of a split-K product; readers add the parts up
// in their order.
#pragma once

#include "common.cuh"

namespace tk {

struct StackedInput {
  const void* x;            // [n_tokens, row_stride] activation type, or null
  const float* parts;       // [n_parts, n_tokens, row_stride] float32, or null
  int n_parts;
  int row_stride;
  long long part_stride;
};

template <typename T>
__device__ __forceinline__ float stacked_ld(const StackedInput& in, size_t off) {
  if (in.parts == nullptr) return to_f32<T>(((const T*)in.x)[off]);
  float acc = 0.0f;
  for (int s = 0; s < in.n_parts; ++s) acc += in.parts[(size_t)s * in.part_stride + off];
  return acc;
}

}  // namespace tk
