// RMS norms whose gain is ONE learned number, for layers that normalise after the residual sum,
// and the learned mix over depth that such a stack may carry.
//
// unit_norm: one block a row.  v = alpha * x + y1 + y2 (float32; y1, y2 optional branch outputs in
//   the run dtype), n = v / sqrt(mean(v^2) + eps) * g.  Outputs, each optional: the sum v (float32),
//   n (float32), and with a depth mix m = sum_{j < n_prev} w[j] X_j + w[n_prev] n over the earlier
//   results X_j of the stack (float32 [.., T, d], one stride apart), in float32; and a copy of the
//   last of these (m if mixed, else n) in the run dtype, which is what the next product reads.  With
//   row_index, output row r is made from batch row row_index[r] (the final norm on the wanted rows).
// embedding_unit_norm: the same norm applied to a gathered embedding row.
// Statistics, sums and the mix are float32; every output is rounded once on store.
#include "common.cuh"
#include "pdl.cuh"

using namespace pbe;

namespace {

// four consecutive elements, 16-byte aligned for float and 8-byte aligned for bfloat16
__device__ __forceinline__ void load4(const float* p, float (&a)[4]) {
  const float4 v = *reinterpret_cast<const float4*>(p);
  a[0] = v.x; a[1] = v.y; a[2] = v.z; a[3] = v.w;
}
__device__ __forceinline__ void load4(const __nv_bfloat16* p, float (&a)[4]) {
  const uint2 raw = *reinterpret_cast<const uint2*>(p);
  const __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
  const __nv_bfloat162 hi = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
  a[0] = __low2float(lo); a[1] = __high2float(lo); a[2] = __low2float(hi); a[3] = __high2float(hi);
}
__device__ __forceinline__ void store4(float* p, const float (&a)[4]) {
  *reinterpret_cast<float4*>(p) = make_float4(a[0], a[1], a[2], a[3]);
}
__device__ __forceinline__ void store4(__nv_bfloat16* p, const float (&a)[4]) {
  __nv_bfloat162 lo = __floats2bfloat162_rn(a[0], a[1]);
  __nv_bfloat162 hi = __floats2bfloat162_rn(a[2], a[3]);
  uint2 raw;
  raw.x = *reinterpret_cast<unsigned*>(&lo);
  raw.y = *reinterpret_cast<unsigned*>(&hi);
  *reinterpret_cast<uint2*>(p) = raw;
}

struct UnitNormParams {
  const float* x;            // [T, d]
  const void* y1;            // [T, d] or null
  const void* y2;            // [T, d] or null
  float alpha;
  const float* gain;         // one number
  float eps;
  float* sum_out;            // [T, d] or null: alpha * x + y1 + y2
  float* normed;             // [T, d] or null
  const float* history;      // X_0: [T, d]; X_j lies j * history_stride floats further
  long long history_stride;
  int n_prev;                // earlier results that enter the mix (0 with mix == null)
  const float* mix;          // [n_prev + 1] or null: no mix
  float* mixed;              // [T, d] or null
  void* lp;                  // [rows, d] in the run dtype or null
  const int32_t* row_index;  // [rows] or null
  int d;
};

template <typename TD, typename TO>
__global__ void unit_norm_kernel(UnitNormParams p) {
  __shared__ float red[33];
  extern __shared__ __align__(16) float row[];
  pdl_launch_dependents();
  const float g = p.gain[0];              // a weight: read ahead of the wait
  pdl_wait();
  const int r = blockIdx.x;
  const int src = p.row_index ? p.row_index[r] : r;
  const int d = p.d;
  const float* x = p.x + (size_t)src * d;
  const TD* y1 = p.y1 ? (const TD*)p.y1 + (size_t)src * d : nullptr;
  const TD* y2 = p.y2 ? (const TD*)p.y2 + (size_t)src * d : nullptr;
  float ss = 0.f;
  float* sum_out = p.sum_out ? p.sum_out + (size_t)src * d : nullptr;
  float* normed = p.normed ? p.normed + (size_t)r * d : nullptr;
  float* mixed = p.mixed ? p.mixed + (size_t)r * d : nullptr;
  TO* lp = p.lp ? (TO*)p.lp + (size_t)r * d : nullptr;
  const float* hist = p.history ? p.history + (size_t)src * d : nullptr;
  if ((d & 3) == 0 && (p.history_stride & 3) == 0) {
    // four elements a thread: 16-byte accesses of the float32 tensors, 8-byte ones of the bfloat16
    for (int i = threadIdx.x * 4; i < d; i += blockDim.x * 4) {
      float v[4], a[4];
      load4(x + i, v);
#pragma unroll
      for (int k = 0; k < 4; ++k) v[k] *= p.alpha;
      if (y1) {
        load4(y1 + i, a);
#pragma unroll
        for (int k = 0; k < 4; ++k) v[k] += a[k];
      }
      if (y2) {
        load4(y2 + i, a);
#pragma unroll
        for (int k = 0; k < 4; ++k) v[k] += a[k];
      }
      store4(row + i, v);
#pragma unroll
      for (int k = 0; k < 4; ++k) ss = fmaf(v[k], v[k], ss);
    }
    const float inv = 1.0f / sqrtf(block_sum(ss, red) / (float)d + p.eps);
    for (int i = threadIdx.x * 4; i < d; i += blockDim.x * 4) {
      float v[4], n[4];
      load4(row + i, v);
      if (sum_out) store4(sum_out + i, v);
#pragma unroll
      for (int k = 0; k < 4; ++k) n[k] = (v[k] * inv) * g;
      if (normed) store4(normed + i, n);
      if (p.mix) {
        float m[4] = {0.f, 0.f, 0.f, 0.f}, h[4];
        for (int j = 0; j < p.n_prev; ++j) {
          const float w = p.mix[j];
          load4(hist + (size_t)j * p.history_stride + i, h);
#pragma unroll
          for (int k = 0; k < 4; ++k) m[k] = fmaf(w, h[k], m[k]);
        }
        const float w = p.mix[p.n_prev];
#pragma unroll
        for (int k = 0; k < 4; ++k) n[k] = fmaf(w, n[k], m[k]);
        if (mixed) store4(mixed + i, n);
      }
      if (lp) store4(lp + i, n);
    }
    return;
  }
  for (int i = threadIdx.x; i < d; i += blockDim.x) {
    float v = p.alpha * x[i];
    if (y1) v += to_float(y1[i]);
    if (y2) v += to_float(y2[i]);
    row[i] = v;
    ss = fmaf(v, v, ss);
  }
  const float inv = 1.0f / sqrtf(block_sum(ss, red) / (float)d + p.eps);
  for (int i = threadIdx.x; i < d; i += blockDim.x) {
    const float v = row[i];
    if (sum_out) sum_out[i] = v;
    const float n = (v * inv) * g;
    if (normed) normed[i] = n;
    float last = n;
    if (p.mix) {
      float m = 0.f;
      for (int j = 0; j < p.n_prev; ++j) m = fmaf(p.mix[j], hist[(size_t)j * p.history_stride + i], m);
      last = fmaf(p.mix[p.n_prev], n, m);
      if (mixed) mixed[i] = last;
    }
    if (lp) lp[i] = from_float<TO>(last);
  }
}

template <typename TW, typename TO>
__global__ void embedding_unit_norm_kernel(float* __restrict__ out, TO* __restrict__ lp, const TW* __restrict__ table,
                                           const int32_t* __restrict__ ids, const float* __restrict__ gain, int d,
                                           int vocab, float eps) {
  __shared__ float red[33];
  extern __shared__ __align__(16) float row[];
  pdl_launch_dependents();
  const float g = gain[0];
  pdl_wait();
  const int t = blockIdx.x;
  const int id = ids[t];
  const bool ok = id >= 0 && id < vocab;  // the host rejects other ids before launch; never read outside the table
  const TW* e = table + (size_t)(ok ? id : 0) * d;
  float ss = 0.f;
  for (int i = threadIdx.x; i < d; i += blockDim.x) {
    const float v = ok ? to_float(e[i]) : 0.f;
    row[i] = v;
    ss = fmaf(v, v, ss);
  }
  const float inv = 1.0f / sqrtf(block_sum(ss, red) / (float)d + eps);
  for (int i = threadIdx.x; i < d; i += blockDim.x) {
    const float n = (row[i] * inv) * g;
    out[(size_t)t * d + i] = n;
    if (lp) lp[(size_t)t * d + i] = from_float<TO>(n);
  }
}

template <typename K>
inline void opt_in(K kernel, size_t smem) {
  if (smem > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
}
}  // namespace

PBE_EXPORT int pbe_unit_norm(const float* x, const void* y1, const void* y2, int y_dtype, float alpha, const float* gain,
                             float eps, float* sum_out, float* normed, const float* history, long long history_stride,
                             int n_prev, const float* mix, float* mixed, void* lp, int lp_dtype,
                             const int32_t* row_index, int rows, int d, cudaStream_t stream) {
  if (rows <= 0) return 0;
  const size_t smem = (size_t)d * sizeof(float);
  if (d < 1 || smem > 200 * 1024 || n_prev < 0 || (mix && n_prev > 0 && !history)) return (int)cudaErrorInvalidValue;
  UnitNormParams p{x, y1, y2, alpha, gain, eps, sum_out, normed, history, history_stride, mix ? n_prev : 0, mix, mixed,
                   lp, row_index, d};
  const int threads = d >= 4096 ? 512 : (d >= 1024 ? 256 : 128);
#define PBE_UN(TD, TO)                                                        \
  do {                                                                        \
    opt_in(unit_norm_kernel<TD, TO>, smem);                                   \
    launch_k(unit_norm_kernel<TD, TO>, rows, threads, smem, stream, p);       \
  } while (0)
  if (y_dtype == PBE_F32 && lp_dtype == PBE_F32) PBE_UN(float, float);
  else if (y_dtype == PBE_BF16 && lp_dtype == PBE_BF16) PBE_UN(__nv_bfloat16, __nv_bfloat16);
  else if (y_dtype == PBE_F32) PBE_UN(float, __nv_bfloat16);
  else PBE_UN(__nv_bfloat16, float);
#undef PBE_UN
  return launch_status();
}

PBE_EXPORT int pbe_embedding_unit_norm(float* out, void* lp, int lp_dtype, const void* table, int table_dtype,
                                       const int32_t* ids, const float* gain, int num_tokens, int d, int vocab, float eps,
                                       cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  const size_t smem = (size_t)d * sizeof(float);
  if (d < 1 || smem > 200 * 1024) return (int)cudaErrorInvalidValue;
  const int threads = d >= 2048 ? 512 : (d >= 512 ? 256 : 128);
#define PBE_EN(TW, TO)                                                                                             \
  do {                                                                                                             \
    opt_in(embedding_unit_norm_kernel<TW, TO>, smem);                                                              \
    launch_k(embedding_unit_norm_kernel<TW, TO>, num_tokens, threads, smem, stream, out, (TO*)lp, (const TW*)table, \
             ids, gain, d, vocab, eps);                                                                            \
  } while (0)
  if (table_dtype == PBE_F32 && lp_dtype == PBE_F32) PBE_EN(float, float);
  else if (table_dtype == PBE_BF16 && lp_dtype == PBE_BF16) PBE_EN(__nv_bfloat16, __nv_bfloat16);
  else if (table_dtype == PBE_F32) PBE_EN(float, __nv_bfloat16);
  else PBE_EN(__nv_bfloat16, float);
#undef PBE_EN
  return launch_status();
}
