// What the masked attention kernels (float32 arithmetic and tensor cores) share: the options of a
// launch, the first key a row sees under each mask, the sink's term and the gate's sigmoid.
#pragma once
#include <cuda_runtime.h>
#include <math.h>

namespace pbe {

struct MaskedExtra {
  const float* bias;         // [H, bias_rows] by head and distance, or null
  int bias_rows;
  int mask_kind;             // 0: all earlier keys, 1: the last `window` keys, 2: the row's chunk of `window` positions
  int unit_sink;
  const void* gate;          // [T, ldg] in the cache's dtype, column head * E + e, or null
  int ldg;
  int D, E;
  int gate_pairs = 0;        // the gate's rows start on 4-byte boundaries: two values a load (tensor-core kernel)
};

__device__ __forceinline__ int first_visible(int pos, int mask_kind, int window) {
  if (mask_kind == 1) return max(0, pos - window + 1);
  if (mask_kind == 2) return (pos / window) * window;
  return 0;
}

__device__ __forceinline__ float sigmoidf_(float x) { return 1.0f / (1.0f + expf(-x)); }

// the sink's term joins (m, l, acc scale): afterwards l includes e^(0 - m') and m' = max(m, 0)
__device__ __forceinline__ void add_unit_sink(float& m, float& l, float& rescale) {
  const float m2 = fmaxf(m, 0.f);
  rescale = m == -INFINITY ? 0.f : expf(m - m2);
  l = l * rescale + expf(-m2);
  m = m2;
}

}  // namespace pbe
