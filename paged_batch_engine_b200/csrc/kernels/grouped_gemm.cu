// Many small matrix products in one launch on the tensor cores (mma.sync m16n8k16, bfloat16
// operands, float32 sums): out_g = A_g W_g^T for groups g that differ in their weights.
//
// Two ways to say which rows belong to which group:
//  * heads:  every row takes part in every group; group g reads columns g * a_group .. of A and
//            writes columns g * out_group .. of the output (the per-head maps of an attention
//            whose keys and values are kept as one latent);
//  * runs:   the rows are sorted by group, every group's run padded to whole row tiles; a tile list
//            names each tile's group, first row and rows (the experts of a routed feed-forward);
//            tiles beyond the list's live part carry group -1.
// W_g is addressed as w[g * w_group + k * wk + n * wn], so both [N, K] and [K, N] matrices are
// read as they lie.  A may be float32 (rounded to bfloat16 as it is staged).  Sums run over K in
// one fixed order, so a row's result does not depend on the other rows.
//
// Epilogues of the heads form: a sigmoid gate per (row, group), and a tail of `rot` values copied
// from behind A's K columns to behind the output's N columns, rotated by the rows' positions
// (pairs (2i, 2i + 1) of its first rot_dims values).
#include "common.cuh"
#include "pdl.cuh"

using namespace pbe;

namespace {
constexpr int GG_BM = 64, GG_BN = 128, GG_BK = 32, GG_PAD = 8;

struct GroupGemmParams {
  const void* a;
  int lda;
  long long a_group;
  const __nv_bfloat16* w;
  long long w_group;
  int wk, wn;
  void* out;
  int ldo;
  long long out_group;
  int T, K, N, groups;
  const int32_t* tiles;      // [n, 3]: group (-1: idle), first row, rows; null: the heads form
  const __nv_bfloat16* gate; // [T, ldg] or null
  int ldg;
  int rot, rot_dims;
  const float* inv_freq;
  const int32_t* positions;
  float rot_scale;           // cos and sin of the tail's rotation are both multiplied by it
  int gate_each;             // the gate has a value per output column: gate[t * ldg + g * N + n]
};

__device__ __forceinline__ void mma16816(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ __nv_bfloat16 as_bf16(float v) { return __float2bfloat16_rn(v); }
__device__ __forceinline__ __nv_bfloat16 as_bf16(__nv_bfloat16 v) { return v; }

__device__ __forceinline__ void ldmatrix_x4(unsigned (&r)[4], const __nv_bfloat16* row) {
  const unsigned addr = (unsigned)__cvta_generic_to_shared(row);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}

// A block of four warps makes a 64 x 128 tile of the output, every warp a 32 x 64 corner of it; the
// operands of the next 32 values of K wait in registers while the current ones are multiplied out of
// shared memory (two buffers, one barrier a step); fragments come by ldmatrix.
template <typename TA, typename TO>
__global__ void __launch_bounds__(128) grouped_gemm_kernel(GroupGemmParams p) {
  constexpr int STR = GG_BK + GG_PAD;
  __shared__ __align__(16) __nv_bfloat16 As[2][GG_BM][STR];
  __shared__ __align__(16) __nv_bfloat16 Ws[2][GG_BN][STR];
  pdl_launch_dependents();
  pdl_wait();
  int g, row0, rows;
  if (p.tiles) {
    const int32_t* tile = p.tiles + (size_t)blockIdx.x * 3;
    g = tile[0]; row0 = tile[1]; rows = tile[2];
    if (g < 0) return;
  } else {
    g = blockIdx.y;
    row0 = blockIdx.x * GG_BM;
    rows = min(GG_BM, p.T - row0);
  }
  const int n0 = blockIdx.z * GG_BN;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g8 = lane >> 2, q2 = (lane & 3) * 2;
  const int wm = (warp >> 1) * 32, wn0 = (warp & 1) * 64;      // the warp's 32 x 64 corner of the tile
  const TA* a = (const TA*)p.a + (size_t)g * p.a_group;
  const __nv_bfloat16* w = p.w + (size_t)g * p.w_group;
  float acc[2][8][4];
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[i][j][0] = acc[i][j][1] = acc[i][j][2] = acc[i][j][3] = 0.f;
  const bool a_vec = (p.lda % 8 == 0) && (p.a_group % 8 == 0) && ((uintptr_t)p.a % 16 == 0);
  const bool w_vec = ((p.wk == 1 ? p.wn : p.wk) % 8 == 0) && (p.w_group % 8 == 0) && ((uintptr_t)p.w % 16 == 0);
  constexpr int A_PER = GG_BM * (GG_BK / 8) / 128;             // 16-byte pieces a thread stages: 2 of A
  constexpr int W_PER = GG_BN * (GG_BK / 8) / 128;             // and 4 of W
  uint4 ra[A_PER], rw[W_PER];
  auto fetch = [&](int k0) {
#pragma unroll
    for (int x = 0; x < A_PER; ++x) {
      const int idx = tid + x * 128;
      const int i = idx >> 2, k = k0 + (idx & 3) * 8;
      __nv_bfloat16 v[8];
      const TA* src = a + (size_t)(row0 + i) * p.lda + k;
      if (i < rows && k + 8 <= p.K && a_vec) {
        if (sizeof(TA) == 2) {
          *reinterpret_cast<uint4*>(v) = *reinterpret_cast<const uint4*>(src);
        } else {
          const float4 x0 = *reinterpret_cast<const float4*>(src), x1 = *reinterpret_cast<const float4*>(src + 4);
          v[0] = as_bf16(x0.x); v[1] = as_bf16(x0.y); v[2] = as_bf16(x0.z); v[3] = as_bf16(x0.w);
          v[4] = as_bf16(x1.x); v[5] = as_bf16(x1.y); v[6] = as_bf16(x1.z); v[7] = as_bf16(x1.w);
        }
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = (i < rows && k + j < p.K) ? as_bf16(src[j]) : as_bf16(0.f);
      }
      ra[x] = *reinterpret_cast<const uint4*>(v);
    }
#pragma unroll
    for (int x = 0; x < W_PER; ++x) {
      const int idx = tid + x * 128;
      __nv_bfloat16 v[8];
      if (p.wk == 1) {                     // [N, K]: eight values of K of one output column
        const int n = idx >> 2, k = k0 + (idx & 3) * 8;
        const __nv_bfloat16* src = w + (size_t)(n0 + n) * p.wn + k;
        if (n0 + n < p.N && k + 8 <= p.K && w_vec) {
          *reinterpret_cast<uint4*>(v) = *reinterpret_cast<const uint4*>(src);
        } else {
#pragma unroll
          for (int j = 0; j < 8; ++j) v[j] = (n0 + n < p.N && k + j < p.K) ? src[j] : as_bf16(0.f);
        }
      } else {                             // [K, N]: eight output columns of one value of K
        const int k = idx >> 4, nc = (idx & 15) * 8;
        const __nv_bfloat16* src = w + (size_t)(k0 + k) * p.wk + (size_t)(n0 + nc) * p.wn;
        if (k0 + k < p.K && n0 + nc + 8 <= p.N && w_vec && p.wn == 1) {
          *reinterpret_cast<uint4*>(v) = *reinterpret_cast<const uint4*>(src);
        } else {
#pragma unroll
          for (int j = 0; j < 8; ++j)
            v[j] = (k0 + k < p.K && n0 + nc + j < p.N) ? src[(size_t)j * p.wn] : as_bf16(0.f);
        }
      }
      rw[x] = *reinterpret_cast<const uint4*>(v);
    }
  };
  auto stash = [&](int buf) {
#pragma unroll
    for (int x = 0; x < A_PER; ++x) {
      const int idx = tid + x * 128;
      *reinterpret_cast<uint4*>(&As[buf][idx >> 2][(idx & 3) * 8]) = ra[x];
    }
#pragma unroll
    for (int x = 0; x < W_PER; ++x) {
      const int idx = tid + x * 128;
      if (p.wk == 1) {
        *reinterpret_cast<uint4*>(&Ws[buf][idx >> 2][(idx & 3) * 8]) = rw[x];
      } else {
        const int k = idx >> 4, nc = (idx & 15) * 8;
        const __nv_bfloat16* v = reinterpret_cast<const __nv_bfloat16*>(&rw[x]);
#pragma unroll
        for (int j = 0; j < 8; ++j) Ws[buf][nc + j][k] = v[j];
      }
    }
  };
  fetch(0);
  stash(0);
  __syncthreads();
  int buf = 0;
  for (int k0 = 0; k0 < p.K; k0 += GG_BK, buf ^= 1) {
    const bool more = k0 + GG_BK < p.K;
    if (more) fetch(k0 + GG_BK);
#pragma unroll
    for (int kk = 0; kk < GG_BK; kk += 16) {
      unsigned af[2][4], bf[4][4];
#pragma unroll
      for (int i = 0; i < 2; ++i)
        ldmatrix_x4(af[i], &As[buf][wm + i * 16 + (lane & 7) + ((lane >> 3) & 1) * 8][kk + (lane >> 4) * 8]);
#pragma unroll
      for (int j = 0; j < 4; ++j)       // two tiles of eight columns a load: {b0, b1} of the first, then of the second
        ldmatrix_x4(bf[j], &Ws[buf][wn0 + j * 16 + (lane & 7) + (lane >> 4) * 8][kk + ((lane >> 3) & 1) * 8]);
#pragma unroll
      for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          mma16816(acc[i][2 * j], af[i], bf[j][0], bf[j][1]);
          mma16816(acc[i][2 * j + 1], af[i], bf[j][2], bf[j][3]);
        }
    }
    if (more) stash(buf ^ 1);          // the other buffer: its readers passed the barrier of the step before
    __syncthreads();
  }
  TO* out = (TO*)p.out + (size_t)g * p.out_group;
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
      const int r = wm + i * 16 + g8 + 8 * hh;
      if (r >= rows) continue;
      const int t = row0 + r;
      float gate = 1.f;
      if (p.gate && !p.gate_each) gate = 1.0f / (1.0f + expf(-__bfloat162float(p.gate[(size_t)t * p.ldg + g])));
      const __nv_bfloat16* gates = p.gate_each ? p.gate + (size_t)t * p.ldg + (size_t)g * p.N : nullptr;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int n = n0 + wn0 + j * 8 + q2;
        float g0 = gate, g1 = gate;
        if (gates) {
          if (n < p.N) g0 = 1.0f / (1.0f + expf(-__bfloat162float(gates[n])));
          if (n + 1 < p.N) g1 = 1.0f / (1.0f + expf(-__bfloat162float(gates[n + 1])));
        }
        if (n < p.N) out[(size_t)t * p.ldo + n] = from_float<TO>(acc[i][j][2 * hh] * g0);
        if (n + 1 < p.N) out[(size_t)t * p.ldo + n + 1] = from_float<TO>(acc[i][j][2 * hh + 1] * g1);
      }
    }
  if (p.rot > 0 && blockIdx.z == 0) {
    for (int idx = tid; idx < rows * (p.rot / 2); idx += 128) {
      const int i = idx / (p.rot / 2), pr = idx - i * (p.rot / 2);
      const int t = row0 + i;
      const TA* src = a + (size_t)t * p.lda + p.K;
      const float u = to_float(src[2 * pr]), v = to_float(src[2 * pr + 1]);
      float x = u, y = v;
      if (2 * pr + 1 < p.rot_dims) {
        float sn, cs;
        sincosf((float)p.positions[t] * p.inv_freq[pr], &sn, &cs);
        sn *= p.rot_scale;
        cs *= p.rot_scale;
        x = u * cs - v * sn;
        y = v * cs + u * sn;
      }
      TO* dst = out + (size_t)t * p.ldo + p.N;
      dst[2 * pr] = from_float<TO>(x);
      dst[2 * pr + 1] = from_float<TO>(y);
    }
  }
}

// The tile list of rows sorted by group, every group's run padded to whole tiles: from the groups'
// row counts.  start[g]: first row of group g's run; tiles[i] = (group, first row, rows), idle
// entries (group -1) up to max_tiles.  One thread: a few hundred entries at most.
__global__ void run_tiles_kernel(const int32_t* __restrict__ counts, int groups, int max_tiles,
                                 int32_t* __restrict__ start, int32_t* __restrict__ tiles) {
  pdl_launch_dependents();
  pdl_wait();
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  int row = 0, n = 0;
  for (int g = 0; g < groups; ++g) {
    start[g] = row;
    for (int left = counts[g]; left > 0 && n < max_tiles; left -= GG_BM, ++n) {
      tiles[n * 3] = g;
      tiles[n * 3 + 1] = row;
      tiles[n * 3 + 2] = left < GG_BM ? left : GG_BM;
      row += GG_BM;
    }
  }
  for (; n < max_tiles; ++n) {
    tiles[n * 3] = -1;
    tiles[n * 3 + 1] = 0;
    tiles[n * 3 + 2] = 0;
  }
}
}  // namespace

PBE_EXPORT int pbe_grouped_gemm_tile_rows() { return GG_BM; }

PBE_EXPORT int pbe_grouped_gemm(const void* a, int a_dtype, int lda, long long a_group, const void* w, long long w_group,
                                int wk, int wn, void* out, int out_dtype, int ldo, long long out_group, int T, int K,
                                int N, int groups, const int32_t* tiles, int num_tiles, const void* gate, int ldg,
                                int rot, int rot_dims, const float* inv_freq, const int32_t* positions,
                                float rot_scale, int gate_each, cudaStream_t stream) {
  if (groups <= 0 || (tiles == nullptr && T <= 0) || (tiles != nullptr && num_tiles <= 0)) return 0;
  GroupGemmParams p{a, lda, a_group, (const __nv_bfloat16*)w, w_group, wk, wn, out, ldo, out_group, T, K, N, groups,
                    tiles, (const __nv_bfloat16*)gate, ldg, rot, rot_dims, inv_freq, positions, rot_scale,
                    gate_each};
  int nz = (N + GG_BN - 1) / GG_BN;
  if (nz == 0) nz = 1;
  dim3 grid = tiles ? dim3(num_tiles, 1, nz) : dim3((T + GG_BM - 1) / GG_BM, groups, nz);
  if (a_dtype == PBE_F32 && out_dtype == PBE_F32) launch_k(grouped_gemm_kernel<float, float>, grid, 128, 0, stream, p);
  else if (a_dtype == PBE_F32) launch_k(grouped_gemm_kernel<float, __nv_bfloat16>, grid, 128, 0, stream, p);
  else if (out_dtype == PBE_F32) launch_k(grouped_gemm_kernel<__nv_bfloat16, float>, grid, 128, 0, stream, p);
  else launch_k(grouped_gemm_kernel<__nv_bfloat16, __nv_bfloat16>, grid, 128, 0, stream, p);
  return launch_status();
}

PBE_EXPORT int pbe_run_tiles(const int32_t* counts, int groups, int max_tiles, int32_t* start, int32_t* tiles,
                             cudaStream_t stream) {
  if (groups <= 0 || max_tiles <= 0) return 0;
  launch_k(run_tiles_kernel, 1, 32, 0, stream, counts, groups, max_tiles, start, tiles);
  return launch_status();
}
