// A gated diagonal linear recurrence (the real-gated linear recurrent unit): per channel c
//
//     r = sigmoid(R_b u_b + c_r),  i = sigmoid(I_b u_b + c_i)        (block-diagonal maps: channel c's block b)
//     log a = -rate * r * softplus(lam_c),  a = exp(log a)
//     S_t = a_t S_(t-1) + sqrt(1 - a_t^2) * i_t * u_t,   out_t = S_t * act(y_t)
//
// with S (float32 [C] per request slot) carried from step to step.
//
// recurrence_gates: the two block-diagonal products in float32 FMAs (the gates enter the recurrence, so
//   they are 32-bit quantities), a tile of 32 rows x 64 channels a block, four rows x two channels x
//   two maps a thread; the epilogue turns them into the recurrence's coefficients a and
//   b = sqrt(1 - a^2) i u, float32 [T, C] each.  1 - a^2 is taken as -expm1(2 log a): exact where a
//   is close to one.
//   Where the input and the maps are bfloat16 the products may instead run on the tensor cores (every
//   product of two bfloat16 numbers is exact in float32 and the sums are float32): the scan then
//   takes the gates' pre-activations z = [R_b u_b | I_b u_b] and forms a and b itself, row by row.
// gated_scan: a thread a channel walks an item's rows in order.  An item is (first row, rows, state
//   from, state to); a place is a state row (>= 0), nothing (-1: start from zero / keep nothing) or
//   scratch entry -(v + 2).  A step's requests are the items themselves (items == null), or, for long
//   portions, chunks side by side: every chunk but a request's last first runs from zero and leaves
//   its end value and the product of its a (first pass), chunk_starts turns these into each chunk's
//   start value, and the second pass runs every chunk from its start and writes the outputs.
#include "common.cuh"
#include "pdl.cuh"

using namespace pbe;

namespace {
constexpr int GT_M = 32, GT_N = 64, GT_K = 32;

struct GateParams {
  const void* u;             // [T, ldu]: the recurrence's input, channel c at column c
  int ldu;
  const void* w_r;           // [B, n, n] ([out, in]) recurrence gate
  const void* w_i;           // [B, n, n] input gate
  const float* b_r;          // [C]
  const float* b_i;          // [C]
  const float* lam;          // [C]
  float rate;
  float* a;                  // [T, C]
  float* b;                  // [T, C]
  int T, C, n;               // n = C / B channels a block
};

__device__ __forceinline__ float softplus_f(float x) { return x > 20.f ? x : log1pf(expf(x)); }
__device__ __forceinline__ float sigmoid_f(float x) { return 1.0f / (1.0f + expf(-x)); }

template <typename TU, typename TW>
__global__ void __launch_bounds__(256) recurrence_gates_kernel(GateParams p) {
  __shared__ float Us[GT_M][GT_K + 1];
  __shared__ float Wr[GT_K][GT_N + 2];
  __shared__ float Wi[GT_K][GT_N + 2];
  pdl_launch_dependents();
  pdl_wait();
  const int blk = blockIdx.y, n = p.n;
  const int t0 = blockIdx.x * GT_M, c0 = blockIdx.z * GT_N;     // c0: first channel of the tile inside its block
  const int tid = threadIdx.x;
  const int cp = tid & 31, rg = tid >> 5;                        // channel pair, group of four rows
  const TU* u = (const TU*)p.u + (size_t)blk * n;
  const TW* wr = (const TW*)p.w_r + (size_t)blk * n * n;
  const TW* wi = (const TW*)p.w_i + (size_t)blk * n * n;
  float ar[4][2], ai[4][2];
#pragma unroll
  for (int j = 0; j < 4; ++j) ar[j][0] = ar[j][1] = ai[j][0] = ai[j][1] = 0.f;
  for (int k0 = 0; k0 < n; k0 += GT_K) {
    for (int idx = tid; idx < GT_M * GT_K; idx += 256) {
      const int i = idx / GT_K, k = idx - i * GT_K;
      const int t = t0 + i;
      Us[i][k] = (t < p.T && k0 + k < n) ? to_float(u[(size_t)t * p.ldu + k0 + k]) : 0.f;
    }
    for (int idx = tid; idx < GT_N * GT_K; idx += 256) {
      const int o = idx / GT_K, k = idx - o * GT_K;              // the maps are [out, in]: k runs fastest
      const bool in = c0 + o < n && k0 + k < n;
      const size_t at = (size_t)(c0 + o) * n + k0 + k;
      Wr[k][o] = in ? to_float(wr[at]) : 0.f;
      Wi[k][o] = in ? to_float(wi[at]) : 0.f;
    }
    __syncthreads();
#pragma unroll 8
    for (int k = 0; k < GT_K; ++k) {
      const float r0 = Wr[k][2 * cp], r1 = Wr[k][2 * cp + 1], i0 = Wi[k][2 * cp], i1 = Wi[k][2 * cp + 1];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float x = Us[rg * 4 + j][k];
        ar[j][0] = fmaf(x, r0, ar[j][0]); ar[j][1] = fmaf(x, r1, ar[j][1]);
        ai[j][0] = fmaf(x, i0, ai[j][0]); ai[j][1] = fmaf(x, i1, ai[j][1]);
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int e = 0; e < 2; ++e) {
    const int cin = c0 + 2 * cp + e;
    if (cin >= n) continue;
    const int c = blk * n + cin;
    const float sp = softplus_f(p.lam[c]), br = p.b_r[c], bi = p.b_i[c];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int t = t0 + rg * 4 + j;
      if (t >= p.T) continue;
      const float r = sigmoid_f(ar[j][e] + br), g = sigmoid_f(ai[j][e] + bi);
      const float log_a = -p.rate * r * sp;
      const float x = to_float(u[(size_t)t * p.ldu + cin]);
      p.a[(size_t)t * p.C + c] = expf(log_a);
      p.b[(size_t)t * p.C + c] = sqrtf(-expm1f(2.0f * log_a)) * g * x;
    }
  }
}

// ------------------------------------------------------------------------------------------------
struct ScanParams {
  const float* a;            // [T, C], or null: the coefficients are formed from z
  const float* b;            // [T, C]
  const float* z;            // [T, B, 2n]: per block the recurrence gate's n pre-activations, then the input gate's
  const void* u;             // [T, ldu]: the recurrence's input (with z)
  int ldu;
  const float* b_r;          // [C] gate biases and lam (with z)
  const float* b_i;
  const float* lam;
  float rate;
  int n;                     // channels a block (with z)
  const void* y;             // [T, ldy]: the gate branch before its activation, or null
  int ldy;
  void* out;                 // [T, C] or null (first pass)
  float* state;              // [slots, C]
  float* scratch_s;          // [entries, C]
  float* scratch_p;          // [entries, C]
  const int32_t* items;      // [n, 4] or null: the requests themselves
  const int32_t* q_start;    // [R]
  const int32_t* q_len;      // [R]
  const int32_t* slots;      // [R]
  int C;
  int act;                   // 0: none, 1: gelu (tanh form)
  int keep_product;          // first pass: the product of a goes to scratch_p
};

__device__ __forceinline__ float gelu_tanh_f(float z) {
  return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

template <typename T>
__global__ void gated_scan_kernel(ScanParams p) {
  pdl_launch_dependents();
  pdl_wait();
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= p.C) return;
  int first, rows, from, to;
  if (p.items) {
    const int32_t* it = p.items + (size_t)blockIdx.x * 4;
    first = it[0]; rows = it[1]; from = it[2]; to = it[3];
  } else {
    first = p.q_start[blockIdx.x]; rows = p.q_len[blockIdx.x]; from = to = p.slots[blockIdx.x];
  }
  if (rows <= 0) return;                             // a padding request of a captured step
  float S = 0.f;
  if (from >= 0) S = p.state[(size_t)from * p.C + c];
  else if (from < -1) S = p.scratch_s[(size_t)(-(from + 2)) * p.C + c];
  float prod = 1.f;
  const bool from_z = p.a == nullptr;
  const float* a = from_z ? nullptr : p.a + (size_t)first * p.C + c;
  const float* b = from_z ? nullptr : p.b + (size_t)first * p.C + c;
  const int blk = from_z ? c / p.n : 0;
  // block blk's 2n pre-activations start at column blk * 2n: the recurrence gate's, then the input gate's
  const float* zr = from_z ? p.z + (size_t)first * 2 * p.C + (size_t)blk * 2 * p.n + (c - blk * p.n) : nullptr;
  const T* u = from_z ? (const T*)p.u + (size_t)first * p.ldu + c : nullptr;
  float neg_rate_sp = 0.f, br = 0.f, bi = 0.f;
  if (from_z) {
    neg_rate_sp = -p.rate * softplus_f(p.lam[c]);
    br = p.b_r[c];
    bi = p.b_i[c];
  }
  const T* y = p.y ? (const T*)p.y + (size_t)first * p.ldy + c : nullptr;
  T* out = p.out ? (T*)p.out + (size_t)first * p.C + c : nullptr;
#pragma unroll 4
  for (int t = 0; t < rows; ++t) {     // unrolled: the rows' loads do not wait for one another, only S does
    float at, bt;
    if (from_z) {
      const float* zt = zr + (size_t)t * 2 * p.C;
      const float log_a = neg_rate_sp * sigmoid_f(zt[0] + br);
      at = expf(log_a);
      bt = sqrtf(-expm1f(2.0f * log_a)) * sigmoid_f(zt[p.n] + bi) * to_float(u[(size_t)t * p.ldu]);
    } else {
      at = a[(size_t)t * p.C];
      bt = b[(size_t)t * p.C];
    }
    S = fmaf(at, S, bt);
    prod *= at;
    if (out) {
      float v = S;
      if (y) {
        const float z = to_float(y[(size_t)t * p.ldy]);
        v *= p.act == 1 ? gelu_tanh_f(z) : z;
      }
      out[(size_t)t * p.C] = from_float<T>(v);
    }
  }
  if (to >= 0) {
    p.state[(size_t)to * p.C + c] = S;
  } else if (to < -1) {
    p.scratch_s[(size_t)(-(to + 2)) * p.C + c] = S;
    if (p.keep_product) p.scratch_p[(size_t)(-(to + 2)) * p.C + c] = prod;
  }
}

// scan entry (state row, first scratch entry, chunks, rows a chunk): chunk k's scratch entry holds
// what the chunk adds from zero (q_k) and its product of a (P_k); it gets the chunk's start value,
// s_0 = the state row, s_(k+1) = P_k s_k + q_k.  The last chunk left nothing: it only gets its start.
__global__ void chunk_starts_kernel(const int32_t* __restrict__ scan, const float* __restrict__ state,
                                    float* __restrict__ scratch_s, const float* __restrict__ scratch_p, int C) {
  pdl_launch_dependents();
  pdl_wait();
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const int32_t* e = scan + (size_t)blockIdx.x * 4;
  const int slot = e[0], entry = e[1], chunks = e[2];
  float s = state[(size_t)slot * C + c];
  for (int k = 0; k < chunks; ++k) {
    const size_t at = (size_t)(entry + k) * C + c;
    const float q = scratch_s[at], pk = scratch_p[at];
    scratch_s[at] = s;
    if (k + 1 < chunks) s = fmaf(pk, s, q);
  }
}
}  // namespace

PBE_EXPORT int pbe_recurrence_gates(const void* u, int ldu, int u_dtype, const void* w_r, const void* w_i, int w_dtype,
                                    const float* b_r, const float* b_i, const float* lam, float rate, float* a, float* b,
                                    int T, int C, int blocks, cudaStream_t stream) {
  if (T <= 0 || C <= 0) return 0;
  if (blocks < 1 || C % blocks != 0) return (int)cudaErrorInvalidValue;
  const int n = C / blocks;
  GateParams p{u, ldu, w_r, w_i, b_r, b_i, lam, rate, a, b, T, C, n};
  dim3 grid((T + GT_M - 1) / GT_M, blocks, (n + GT_N - 1) / GT_N);
  if (u_dtype == PBE_F32 && w_dtype == PBE_F32) launch_k(recurrence_gates_kernel<float, float>, grid, 256, 0, stream, p);
  else if (u_dtype == PBE_BF16 && w_dtype == PBE_BF16)
    launch_k(recurrence_gates_kernel<__nv_bfloat16, __nv_bfloat16>, grid, 256, 0, stream, p);
  else if (u_dtype == PBE_F32) launch_k(recurrence_gates_kernel<float, __nv_bfloat16>, grid, 256, 0, stream, p);
  else launch_k(recurrence_gates_kernel<__nv_bfloat16, float>, grid, 256, 0, stream, p);
  return launch_status();
}

// mode 0: every request one item (from the step's own arrays); 1: first pass over `items`; 2: second pass.
PBE_EXPORT int pbe_gated_scan(const float* a, const float* b, const float* z, const void* u, int ldu, const float* b_r,
                              const float* b_i, const float* lam, float rate, int n, const void* y, int ldy, void* out,
                              int dtype, float* state,
                              float* scratch_s, float* scratch_p, const int32_t* items, int num_items,
                              const int32_t* q_start, const int32_t* q_len, const int32_t* slots, int C, int act,
                              int mode, cudaStream_t stream) {
  if (num_items <= 0 || C <= 0) return 0;
  if ((mode != 0 && items == nullptr) || (mode == 0 && (q_start == nullptr || q_len == nullptr || slots == nullptr)))
    return (int)cudaErrorInvalidValue;
  if ((a == nullptr) != (z != nullptr) || (z != nullptr && (n < 1 || C % n != 0 || !u || !b_r || !b_i || !lam)))
    return (int)cudaErrorInvalidValue;
  ScanParams p{a, b, z, u, ldu, b_r, b_i, lam, rate, n, mode == 1 ? nullptr : y, ldy, mode == 1 ? nullptr : out, state, scratch_s, scratch_p,
               mode == 0 ? nullptr : items, q_start, q_len, slots, C, act, mode == 1 ? 1 : 0};
  const int threads = C >= 128 ? 128 : 64;
  dim3 grid(num_items, (C + threads - 1) / threads);
  if (dtype == PBE_F32) launch_k(gated_scan_kernel<float>, grid, threads, 0, stream, p);
  else launch_k(gated_scan_kernel<__nv_bfloat16>, grid, threads, 0, stream, p);
  return launch_status();
}

PBE_EXPORT int pbe_chunk_starts(const int32_t* scan, int num_scan, const float* state, float* scratch_s,
                                const float* scratch_p, int C, cudaStream_t stream) {
  if (num_scan <= 0 || C <= 0) return 0;
  const int threads = C >= 128 ? 128 : 64;
  launch_k(chunk_starts_kernel, dim3(num_scan, (C + threads - 1) / threads), threads, 0, stream, scan, state, scratch_s,
           scratch_p, C);
  return launch_status();
}
