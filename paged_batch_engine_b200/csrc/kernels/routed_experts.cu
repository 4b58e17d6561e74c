// A feed-forward made of many small gated experts of which each token uses a few.
//
// route: from float32 router logits [T, E]: scores s = softmax over all experts, or (score_kind 1)
// sigmoid of each logit; the choice is made on c = s + correction (a learned vector, optional);
// experts form `groups` equal groups of neighbours, a group's rank is its largest c or (group_rank
// 2) the sum of its two largest, and only experts of the `keep` best groups can be chosen (groups =
// 1: no restriction; a barred expert is out whatever its c, which may be negative); the `top`
// allowed experts with the largest c are chosen (ties: the lower index); their weights are their
// scores s, without the correction, over the sum of the chosen scores (+ 1e-20), times `scale`.
// One warp per token.
//
// expert_rows: for few rows (decoded tokens).  Per (token, chosen expert) pair the expert's gate
// and up rows are streamed against the token's input (blocks of 32 hidden units, a warp per unit,
// the lanes along the input in 16-byte loads), h = silu(g) * u goes to scratch memory in float32;
// a second launch streams the down rows against it (blocks of 32 output columns) and writes the
// weighted result to the pair's own slot, [T, top, W]; combine adds a token's slots in order, so
// a token's result never depends on what else is in the step.
//
// For many rows the host side sorts the rows by expert (pair_rows / scatter below) and runs one
// matrix product per expert over its rows.
#include "common.cuh"
#include "pdl.cuh"

using namespace pbe;

namespace {
constexpr int MAX_PER_LANE = 16;       // experts a lane holds: up to 512 experts
constexpr int MAX_TOP = 32;

struct RouteParams {
  const float* logits;       // [T, E]
  int32_t* chosen;           // [T, top]
  float* weights;            // [T, top]
  int T, E, top, groups, keep;
  float scale;
  int score_kind;            // 0: softmax over the experts, 1: sigmoid
  const float* correction;   // [E] or null: added to the scores for the choice only
  int group_rank;            // 1: a group's largest choice score, 2: the sum of its two largest
};

// the lane-distributed argmax of v (lane l holds experts l, l + 32, ...); ties go to the lower index
__device__ __forceinline__ void warp_argmax(float& best, int& at) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ob = __shfl_xor_sync(0xffffffffu, best, o);
    const int oa = __shfl_xor_sync(0xffffffffu, at, o);
    if (ob > best || (ob == best && oa < at)) { best = ob; at = oa; }
  }
}

__global__ void route_kernel(RouteParams p) {
  pdl_launch_dependents();
  pdl_wait();
  const int warps = blockDim.x >> 5;
  const int t = blockIdx.x * warps + (threadIdx.x >> 5);
  if (t >= p.T) return;
  const int lane = threadIdx.x & 31, E = p.E;
  const float* z = p.logits + (size_t)t * E;
  float s[MAX_PER_LANE];     // the scores
  float c[MAX_PER_LANE];     // the choice scores
  if (p.score_kind == 1) {
#pragma unroll
    for (int i = 0; i < MAX_PER_LANE; ++i) {
      const int e = lane + 32 * i;
      const float v = e < E ? 1.0f / (1.0f + expf(-z[e])) : 0.f;
      s[i] = v >= 0.f ? v : 0.f;          // not a number (a padding row nobody wrote): counts as 0
    }
  } else {
    float m = -INFINITY;
#pragma unroll
    for (int i = 0; i < MAX_PER_LANE; ++i) {
      const int e = lane + 32 * i;
      s[i] = e < E ? z[e] : -INFINITY;
      m = fmaxf(m, s[i]);
    }
    m = warp_max(m);
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < MAX_PER_LANE; ++i) {
      const int e = lane + 32 * i;
      s[i] = e < E ? expf(s[i] - m) : 0.f;
      sum += s[i];
    }
    sum = warp_sum(sum);
#pragma unroll
    for (int i = 0; i < MAX_PER_LANE; ++i) {
      // a row of logits that are not numbers (a padding row of a captured step, whose input nobody
      // wrote) still chooses experts that exist: its scores count as 0 and the lowest indices win
      const float v = s[i] / sum;
      s[i] = v >= 0.f ? v : 0.f;
    }
  }
#pragma unroll
  for (int i = 0; i < MAX_PER_LANE; ++i) {
    const int e = lane + 32 * i;
    c[i] = s[i] + ((p.correction && e < E) ? p.correction[e] : 0.f);
  }
  // allowed[i]: may expert lane + 32 i still be chosen
  bool allowed[MAX_PER_LANE];
#pragma unroll
  for (int i = 0; i < MAX_PER_LANE; ++i) allowed[i] = lane + 32 * i < E;
  if (p.groups > 1 && p.keep < p.groups) {
    const int per = E / p.groups;
    // rank of group g: in lane g % 32, slot g / 32 (groups <= 64)
    float rank[2] = {-INFINITY, -INFINITY};
    for (int g = 0; g < p.groups; ++g) {
      float best = -INFINITY;
      int at = 0x7fffffff;
#pragma unroll
      for (int i = 0; i < MAX_PER_LANE; ++i) {
        const int e = lane + 32 * i;
        if (e < E && e / per == g && (c[i] > best || (c[i] == best && e < at))) { best = c[i]; at = e; }
      }
      warp_argmax(best, at);
      float value = best;
      if (p.group_rank == 2 && per > 1) {
        float second = -INFINITY;
        int at2 = 0x7fffffff;
#pragma unroll
        for (int i = 0; i < MAX_PER_LANE; ++i) {
          const int e = lane + 32 * i;
          if (e < E && e / per == g && e != at && (c[i] > second || (c[i] == second && e < at2))) {
            second = c[i];
            at2 = e;
          }
        }
        warp_argmax(second, at2);
        value = best + second;
      }
      if (lane == (g & 31)) rank[g >> 5] = value;
    }
    unsigned long long kept_lo = 0ull;          // bit g: group g is kept
    for (int round = 0; round < p.keep; ++round) {
      float best = -INFINITY;
      int at = 0x7fffffff;
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const int g = lane + 32 * j;
        if (g < p.groups && !((kept_lo >> g) & 1ull) && (rank[j] > best || (rank[j] == best && g < at))) {
          best = rank[j];
          at = g;
        }
      }
      warp_argmax(best, at);
      if (at >= p.groups) {                     // nothing compares (ranks that are not numbers): the lowest group left
        at = 0;
        while ((kept_lo >> at) & 1ull) ++at;
      }
      kept_lo |= 1ull << at;
    }
#pragma unroll
    for (int i = 0; i < MAX_PER_LANE; ++i) {
      const int e = lane + 32 * i;
      allowed[i] = e < E && ((kept_lo >> (e / per)) & 1ull);
    }
  }
  float picked_s[MAX_TOP];
  int picked_e[MAX_TOP];
  float total = 0.f;
  for (int k = 0; k < p.top; ++k) {
    float best = -INFINITY, best_s = 0.f;
    int at = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < MAX_PER_LANE; ++i) {
      const int e = lane + 32 * i;
      if (allowed[i] && (at == 0x7fffffff || c[i] > best || (c[i] == best && e < at))) { best = c[i]; at = e; best_s = s[i]; }
    }
    {   // the warp's best: the larger choice score, ties (and lanes with nothing) to the lower index
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int oa = __shfl_xor_sync(0xffffffffu, at, o);
        const float os = __shfl_xor_sync(0xffffffffu, best_s, o);
        const bool take = oa != 0x7fffffff && (at == 0x7fffffff || ob > best || (ob == best && oa < at));
        if (take) { best = ob; at = oa; best_s = os; }
      }
    }
#pragma unroll
    for (int i = 0; i < MAX_PER_LANE; ++i)
      if (lane + 32 * i == at) allowed[i] = false;
    if (k < MAX_TOP) { picked_s[k] = best_s; picked_e[k] = at; }
    total += best_s;
  }
  if (lane == 0) {
    const float inv = p.scale / (total + 1e-20f);
    for (int k = 0; k < p.top && k < MAX_TOP; ++k) {
      p.chosen[(size_t)t * p.top + k] = picked_e[k];
      p.weights[(size_t)t * p.top + k] = picked_s[k] * inv;
    }
  }
}

// ------------------------------------------------------------------------------------------------
struct ExpertRowsParams {
  const void* x;             // [T, W]
  const void* w_gate;        // expert e's [F, W] at element e * gu_stride
  const void* w_up;          // the same (gate and up may lie in one [E, 2F, W] tensor)
  long long gu_stride;
  const void* w_down;        // [E, W, F]
  const int32_t* chosen;     // [T, top]
  const float* weights;      // [T, top]
  float* hidden;             // [T * top, F] scratch: silu(gate) * up of every pair
  float* part;               // [T, top, W]
  int T, W, F, top;
  int act;                   // 0: silu(g) * u; 1: g <- min(g, limit), u <- clamp(u, +-limit), g sigmoid(alpha g) (u + 1)
  float limit, alpha;
};

// dot product of a weight row with a float32 vector in shared memory, the lanes along the row;
// 16-byte loads of the weights where the row allows them (n a multiple of 8 bfloat16 / 4 float)
__device__ __forceinline__ float dot_row(const float* __restrict__ w, const float* __restrict__ x, int n, int lane) {
  float a = 0.f;
  if ((n & 3) == 0 && (((uintptr_t)w) & 15) == 0) {
    for (int i = lane * 4; i < n; i += 128) {
      const float4 v = *reinterpret_cast<const float4*>(w + i);
      a = fmaf(v.x, x[i], a); a = fmaf(v.y, x[i + 1], a); a = fmaf(v.z, x[i + 2], a); a = fmaf(v.w, x[i + 3], a);
    }
  } else {
    for (int i = lane; i < n; i += 32) a = fmaf(w[i], x[i], a);
  }
  return warp_sum(a);
}
__device__ __forceinline__ float dot_row(const __nv_bfloat16* __restrict__ w, const float* __restrict__ x, int n,
                                         int lane) {
  float a = 0.f;
  if ((n & 7) == 0 && (((uintptr_t)w) & 15) == 0) {
    for (int i = lane * 8; i < n; i += 256) {
      const uint4 raw = *reinterpret_cast<const uint4*>(w + i);
      const unsigned u[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u[j]));
        a = fmaf(f.x, x[i + 2 * j], a);
        a = fmaf(f.y, x[i + 2 * j + 1], a);
      }
    }
  } else {
    for (int i = lane; i < n; i += 32) a = fmaf(to_float(w[i]), x[i], a);
  }
  return warp_sum(a);
}

constexpr int ER_WARPS = 8;
constexpr int ER_UNITS = 32;      // hidden units (first kernel) or output columns (second) a block takes

// block (pair, slice of the hidden units): h = silu(W_gate x) * (W_up x) for its units
template <typename T>
__global__ void __launch_bounds__(ER_WARPS * 32) expert_hidden_kernel(ExpertRowsParams p) {
  extern __shared__ __align__(16) float xs[];        // [W]
  pdl_launch_dependents();
  pdl_wait();
  const int pair = blockIdx.x;
  const int t = pair / p.top;
  const int e = p.chosen[pair];
  const T* x = (const T*)p.x + (size_t)t * p.W;
  for (int i = threadIdx.x; i < p.W; i += blockDim.x) xs[i] = to_float(x[i]);
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const T* wg = (const T*)p.w_gate + (size_t)e * p.gu_stride;
  const T* wu = (const T*)p.w_up + (size_t)e * p.gu_stride;
  const int f_end = min(p.F, (blockIdx.y + 1) * ER_UNITS);
  for (int f = blockIdx.y * ER_UNITS + warp; f < f_end; f += ER_WARPS) {
    const float g = dot_row(wg + (size_t)f * p.W, xs, p.W, lane);
    const float u = dot_row(wu + (size_t)f * p.W, xs, p.W, lane);
    if (lane == 0) {
      float h;
      if (p.act == 1) {
        const float gc = fminf(g, p.limit), uc = fminf(fmaxf(u, -p.limit), p.limit);
        h = (gc / (1.0f + expf(-p.alpha * gc))) * (uc + 1.0f);
      } else {
        h = (g / (1.0f + expf(-g))) * u;
      }
      p.hidden[(size_t)pair * p.F + f] = h;
    }
  }
}

// block (pair, slice of the output columns): weight * W_down h for its columns
template <typename T>
__global__ void __launch_bounds__(ER_WARPS * 32) expert_down_kernel(ExpertRowsParams p) {
  extern __shared__ __align__(16) float hs[];        // [F]
  pdl_launch_dependents();
  pdl_wait();
  const int pair = blockIdx.x;
  const int e = p.chosen[pair];
  const float weight = p.weights[pair];
  for (int i = threadIdx.x; i < p.F; i += blockDim.x) hs[i] = p.hidden[(size_t)pair * p.F + i];
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const T* wd = (const T*)p.w_down + (size_t)e * p.W * p.F;
  float* out = p.part + (size_t)pair * p.W;
  const int c_end = min(p.W, (blockIdx.y + 1) * ER_UNITS);
  for (int c = blockIdx.y * ER_UNITS + warp; c < c_end; c += ER_WARPS) {
    const float y = dot_row(wd + (size_t)c * p.F, hs, p.F, lane);
    if (lane == 0) out[c] = weight * y;
  }
}

// `addend` (optional, [T, W]): what every token gets besides its experts (a shared expert's output)
template <typename T>
__global__ void combine_kernel(const float* __restrict__ part, const T* __restrict__ addend, T* __restrict__ out,
                               int top, int W, size_t total) {
  pdl_launch_dependents();
  pdl_wait();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const size_t t = i / W;
    const int c = (int)(i - t * W);
    float a = 0.f;
    for (int k = 0; k < top; ++k) a += part[(t * top + k) * W + c];
    if (addend) a += to_float(addend[i]);
    out[i] = from_float<T>(a);
  }
}

// ------------------------------------------------------------------------------------------------
// Rows sorted by expert: pair (t, k) gets a place in the run of its expert.  counts[e] first
// (count_kernel), then the runs' starts on the host or by a scan, then place_kernel hands the
// places out in (t, k) order inside every expert's run: a single block walks the pairs of an
// expert in order, so the order inside a run is the tokens' own and nothing depends on timing.
__global__ void place_kernel(const int32_t* __restrict__ chosen, int pairs, int E, int32_t* __restrict__ counts,
                             int32_t* __restrict__ place) {
  // block e: places of the pairs that chose expert e, in pair order
  __shared__ int base;
  __shared__ int warp_tot[32];
  const int e = blockIdx.x;
  if (threadIdx.x == 0) base = 0;
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
  for (int i0 = 0; i0 < pairs; i0 += blockDim.x) {
    const int i = i0 + threadIdx.x;
    const bool mine = i < pairs && chosen[i] == e;
    const unsigned ballot = __ballot_sync(0xffffffffu, mine);
    if (lane == 0) warp_tot[warp] = __popc(ballot);
    __syncthreads();
    int before = base;
    for (int w = 0; w < warp; ++w) before += warp_tot[w];
    if (mine) place[i] = before + __popc(ballot & ((1u << lane) - 1u));
    __syncthreads();
    if (threadIdx.x == 0) {
      int tot = 0;
      for (int w = 0; w < warps; ++w) tot += warp_tot[w];
      base += tot;
    }
    __syncthreads();
  }
  if (threadIdx.x == 0) counts[e] = base;
}

// gathered[start[e] + place] = x[t] for every pair; and the way back, weighted:
template <typename T>
__global__ void gather_rows_kernel(const T* __restrict__ x, const int32_t* __restrict__ chosen,
                                   const int32_t* __restrict__ place, const int32_t* __restrict__ start,
                                   T* __restrict__ gathered, int top, int W) {
  const int pair = blockIdx.x;
  const int t = pair / top;
  const size_t dst = (size_t)(start[chosen[pair]] + place[pair]) * W;
  for (int i = threadIdx.x; i < W; i += blockDim.x) gathered[dst + i] = x[(size_t)t * W + i];
}

template <typename T>
__global__ void scatter_rows_kernel(const T* __restrict__ y, const int32_t* __restrict__ chosen,
                                    const int32_t* __restrict__ place, const int32_t* __restrict__ start,
                                    const float* __restrict__ weights, const T* __restrict__ addend,
                                    T* __restrict__ out, int top, int W) {
  const int t = blockIdx.x;
  for (int i = threadIdx.x; i < W; i += blockDim.x) {
    float a = 0.f;
    for (int k = 0; k < top; ++k) {
      const int pair = t * top + k;
      a += weights[pair] * to_float(y[(size_t)(start[chosen[pair]] + place[pair]) * W + i]);
    }
    if (addend) a += to_float(addend[(size_t)t * W + i]);
    out[(size_t)t * W + i] = from_float<T>(a);
  }
}
}  // namespace

PBE_EXPORT int pbe_route(const float* logits, int32_t* chosen, float* weights, int T, int E, int top, int groups,
                         int keep, float scale, int score_kind, const float* correction, int group_rank,
                         cudaStream_t stream) {
  if (T <= 0) return 0;
  if (E < 1 || E > 32 * MAX_PER_LANE || top < 1 || top > MAX_TOP || top > E || groups < 1 || groups > 64 ||
      E % groups != 0 || keep < 1 || keep > groups || top > keep * (E / groups) || score_kind < 0 || score_kind > 1 ||
      group_rank < 1 || group_rank > 2)
    return (int)cudaErrorInvalidValue;
  RouteParams p{logits, chosen, weights, T, E, top, groups, keep, scale, score_kind, correction, group_rank};
  launch_k(route_kernel, (T + 3) / 4, 128, 0, stream, p);
  return launch_status();
}

PBE_EXPORT int pbe_expert_rows(const void* x, const void* w_gate, const void* w_up, long long gu_stride,
                               const void* w_down, const int32_t* chosen, const float* weights, float* hidden,
                               float* part, void* out, int dtype, int T, int W, int F, int top, int act, float limit,
                               float alpha, const void* addend, cudaStream_t stream) {
  if (T <= 0) return 0;
  ExpertRowsParams p{x, w_gate, w_up, gu_stride, w_down, chosen, weights, hidden, part, T, W, F, top, act, limit, alpha};
  const size_t smem1 = sizeof(float) * (size_t)W, smem2 = sizeof(float) * (size_t)F;
  if (smem1 > 200 * 1024 || smem2 > 200 * 1024) return (int)cudaErrorInvalidValue;
  dim3 grid1(T * top, (F + ER_UNITS - 1) / ER_UNITS), grid2(T * top, (W + ER_UNITS - 1) / ER_UNITS);
#define PBE_ER(TT)                                                                                             \
  do {                                                                                                         \
    static size_t opted = 48 * 1024;                                                                           \
    if (smem1 > opted || smem2 > opted) {                                                                      \
      cudaFuncSetAttribute(expert_hidden_kernel<TT>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024); \
      cudaFuncSetAttribute(expert_down_kernel<TT>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);   \
      opted = 200 * 1024;                                                                                      \
    }                                                                                                          \
    launch_k(expert_hidden_kernel<TT>, grid1, ER_WARPS * 32, smem1, stream, p);                                \
    launch_k(expert_down_kernel<TT>, grid2, ER_WARPS * 32, smem2, stream, p);                                  \
  } while (0)
  if (dtype == PBE_F32) PBE_ER(float); else PBE_ER(__nv_bfloat16);
#undef PBE_ER
  int e = launch_status();
  if (e != 0) return e;
  const size_t total = (size_t)T * W;
  size_t blocks = (total + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  if (dtype == PBE_F32)
    launch_k(combine_kernel<float>, (int)blocks, 256, 0, stream, (const float*)part, (const float*)addend, (float*)out,
             top, W, total);
  else
    launch_k(combine_kernel<__nv_bfloat16>, (int)blocks, 256, 0, stream, (const float*)part,
             (const __nv_bfloat16*)addend, (__nv_bfloat16*)out, top, W, total);
  return launch_status();
}

PBE_EXPORT int pbe_expert_places(const int32_t* chosen, int pairs, int E, int32_t* counts, int32_t* place,
                                 cudaStream_t stream) {
  if (pairs <= 0) return 0;
  place_kernel<<<E, 256, 0, stream>>>(chosen, pairs, E, counts, place);
  return launch_status();
}

PBE_EXPORT int pbe_expert_gather(const void* x, const int32_t* chosen, const int32_t* place, const int32_t* start,
                                 void* gathered, int dtype, int T, int top, int W, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (dtype == PBE_F32)
    gather_rows_kernel<float><<<T * top, 128, 0, stream>>>((const float*)x, chosen, place, start, (float*)gathered, top, W);
  else
    gather_rows_kernel<__nv_bfloat16><<<T * top, 128, 0, stream>>>((const __nv_bfloat16*)x, chosen, place, start,
                                                                  (__nv_bfloat16*)gathered, top, W);
  return launch_status();
}

PBE_EXPORT int pbe_expert_scatter(const void* y, const int32_t* chosen, const int32_t* place, const int32_t* start,
                                  const float* weights, void* out, int dtype, int T, int top, int W,
                                  const void* addend, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (dtype == PBE_F32)
    scatter_rows_kernel<float><<<T, 128, 0, stream>>>((const float*)y, chosen, place, start, weights,
                                                     (const float*)addend, (float*)out, top, W);
  else
    scatter_rows_kernel<__nv_bfloat16><<<T, 128, 0, stream>>>((const __nv_bfloat16*)y, chosen, place, start, weights,
                                                             (const __nv_bfloat16*)addend, (__nv_bfloat16*)out, top, W);
  return launch_status();
}
