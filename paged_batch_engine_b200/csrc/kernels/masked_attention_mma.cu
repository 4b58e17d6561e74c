// The masked attention of masked_attention.cu for bfloat16 pages on the tensor cores (mma.sync
// m16n8k16, float32 accumulation), flash style: scores, softmax statistics and the output
// accumulator stay in registers; keys and values stream from the pages through shared memory,
// double buffered with cp.async.  Same options (mask, bias by head and distance, unit sink, gate),
// same work list (request, row tile, key split) and the same partial buffers as the float32 kernel,
// whose merge kernel puts the key splits together.
//
// Scores and softmax weights are float32 quantities and stay so through the tensor cores: the
// float32 query is fed as the sum of two bfloat16 numbers (its rounding and the rounding of what is
// left), and so is every weight in the weighted sum of the values; each product therefore costs two
// mma instructions and carries about 16 bits of the factor instead of 8.  Keys and values are the
// bfloat16 numbers the pages hold.
//
// A block of eight warps takes a tile of BM = 64 packed rows (row x query head of the key/value
// group) and the keys of its split.  Two modes, by the rows the tile really has:
//   rows mode (more than 16): warp w owns rows 16 (w & 3) .. 16 (w & 3) + 15 and visits half w >> 2 of
//   every key tile with softmax statistics of its own; warp w + 4 hands its sums to warp w at the end
//   (two warps a row group: sixteen warps a multiprocessor hide the chain ldmatrix -> mma -> softmax
//   -> mma of a key tile, which eight did not);
//   keys mode (at most 16: decoded tokens): all warps own rows 0 .. 15 and warp w < 4 visits keys
//   16w .. 16w + 15 of every key tile; warp 0 merges the four at the end.
//
// Compile with -DPBE_MA_D=<key width> -DPBE_MA_E=<value width>, multiples of 16 up to 256.
#include <cuda_bf16.h>

#include "attention_params.cuh"
#include "common.cuh"
#include "masked_attention.cuh"
#include "pdl.cuh"

using namespace pbe;

#if !defined(PBE_MA_D) || !defined(PBE_MA_E)
#error "PBE_MA_D and PBE_MA_E must be defined"
#endif

// blocks a multiprocessor the register budget aims at: two (sixteen warps) while the output
// accumulator of a thread stays within 64 registers
#ifndef PBE_MA_BLOCKS
#define PBE_MA_BLOCKS ((PBE_MA_D <= 128 && PBE_MA_E <= 128) ? 2 : 1)
#endif

namespace {
typedef __nv_bfloat16 bf16;
constexpr int D = PBE_MA_D, E = PBE_MA_E;
static_assert(D % 16 == 0 && E % 16 == 0 && D >= 16 && E >= 16 && D <= 256 && E <= 256,
              "head widths are multiples of 16, at most 256");
constexpr int BM = 64;                         // packed rows per block
constexpr int BN = (D + E > 256) ? 32 : 64;    // keys per tile
constexpr int NT = 256;                        // eight warps
constexpr int LDQ = D + 8, LDK = D + 8, LDV = E + 8;   // shared row strides in elements (16-byte rows, no bank conflicts)
constexpr int KSTEPS = D / 16;                 // k-steps of q . k
constexpr int N2L = BN / 32;                   // 16-key score steps a warp takes of a key tile at most (half the tile)
constexpr int SNT = 2 * N2L;                   // its 8-key score tiles
constexpr int ONT = E / 8;                     // 8-wide output tiles
constexpr int Q_ELEMS = BM * LDQ;              // one of the two query arrays
constexpr int STAGE_ELEMS = BN * (LDK + LDV);
constexpr size_t KV_BYTES = 2 * (size_t)STAGE_ELEMS * sizeof(bf16);
constexpr size_t MERGE_BYTES = (size_t)4 * 16 * (E + 2) * sizeof(float);   // up to four warps' partial results
constexpr size_t SMEM_BYTES = 2 * (size_t)Q_ELEMS * sizeof(bf16) + (KV_BYTES > MERGE_BYTES ? KV_BYTES : MERGE_BYTES);

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, bool valid) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  const int bytes = valid ? 16 : 0;            // 0: the 16 bytes are filled with zeros
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}
__device__ __forceinline__ void ldmatrix_x4(unsigned (&r)[4], const void* smem) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void ldmatrix_x4_trans(unsigned (&r)[4], const void* smem) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
// not volatile: a product is a function of its registers alone, so the compiler may order the
// products of different accumulators between one another (two in a row on one accumulator wait for
// each other)
__device__ __forceinline__ void mma_bf16(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
  asm(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// x = hi + lo + (an error of about 2^-17 |x|), both bfloat16:
// two floats as a (hi, hi) and a (lo, lo) pair of bfloat16, the lower index in the lower half; both
// roundings of a pair in one conversion
__device__ __forceinline__ void split_pair(float x, float y, unsigned& hi, unsigned& lo) {
  const __nv_bfloat162 h = __floats2bfloat162_rn(x, y);
  hi = *reinterpret_cast<const unsigned*>(&h);
  const float xh = __uint_as_float(hi << 16), yh = __uint_as_float(hi & 0xffff0000u);
  const __nv_bfloat162 l = __floats2bfloat162_rn(x - xh, y - yh);
  lo = *reinterpret_cast<const unsigned*>(&l);
}

__global__ void __launch_bounds__(NT, PBE_MA_BLOCKS) masked_attention_mma_kernel(AttnParams p, MaskedExtra x) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* Qh = reinterpret_cast<bf16*>(smem_raw);     // [BM][LDQ] the queries' roundings
  bf16* Ql = Qh + Q_ELEMS;                          // and what the roundings left
  bf16* KVs = Ql + Q_ELEMS;                         // stage s: keys [BN][LDK], then values [BN][LDV]

  pdl_launch_dependents();
  pdl_wait();
  const int32_t* work = p.work + (size_t)blockIdx.x * 4;
  const int r = work[0];
  if (r < 0) return;
  const int m_tile = work[1], split = work[2], nsplit = work[3];
  const int kvh = blockIdx.y;
  const int H = p.num_heads, KV = p.num_kv_heads, G = H / KV, P = p.page_tokens;
  const int qs = p.q_start[r], nq = p.q_len[r], sl = p.seq_len[r];
  const int n_packed = nq * G;
  const int pr0 = m_tile * BM;
  if (pr0 >= n_packed) return;
  const int rows_here = min(BM, n_packed - pr0);
  const bool keys_mode = rows_here <= 16;
  const int row_lo = pr0 / G;
  const int row_hi = (pr0 + rows_here - 1) / G;
  const int pos0 = sl - nq;
  const int hi_key = pos0 + row_hi + 1;
  const int lo_key = first_visible(pos0 + row_lo, x.mask_kind, p.window);
  int k_begin = lo_key, k_end = hi_key;
  if (nsplit > 1) {
    // split boundaries are absolute multiples of split_keys, counted from the first split that a
    // window of this size at the request's first row can reach: the work list's own rule
    const int lo_req = x.mask_kind ? max(0, pos0 - p.window + 1) : 0;
    const int s0 = lo_req / p.split_keys;
    k_begin = max(lo_key, (s0 + split) * p.split_keys);
    k_end = min(hi_key, (s0 + split + 1) * p.split_keys);
  }
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  const float* q = (const float*)p.q;
  const bf16* kc = (const bf16*)p.k_cache;
  const bf16* vc = (const bf16*)p.v_cache;
  const int32_t* bt = p.block_table + (size_t)r * p.bt_stride;

  // the first key tile is requested before anything else
  constexpr int TPR = NT / BN;          // threads that share a key's row when a tile is fetched
  const int ld_j = tid / TPR, ld_part = tid - ld_j * TPR;
  // the page of this thread's key in the tile at ts (-1: none); looked up a tile ahead of its use,
  // so that the request for the tile does not wait for the block table
  auto page_of = [&](int ts) -> int {
    const int key = ts + ld_j;
    return (ts < k_end && key >= k_begin && key < k_end) ? bt[key / P] : -1;
  };
  auto load_tile = [&](int stage, int ts, int page) {
    bf16* Ks = KVs + stage * STAGE_ELEMS;
    bf16* Vs = Ks + BN * LDK;
    const int key = ts + ld_j;
    const bool ok = page >= 0;
    const long long b = ok ? ((long long)page * KV + kvh) * P + key % P : 0;
    const bf16* ksrc = kc + b * D;
    const bf16* vsrc = vc + b * E;
    for (int c = ld_part; c < D / 8; c += TPR) cp_async16(Ks + ld_j * LDK + c * 8, ksrc + c * 8, ok);
    for (int c = ld_part; c < E / 8; c += TPR) cp_async16(Vs + ld_j * LDV + c * 8, vsrc + c * 8, ok);
  };

  const int tile0 = (k_begin / BN) * BN;
  int page_next = page_of(tile0);
  if (tile0 < k_end) load_tile(0, tile0, page_next);
  cp_async_commit();
  page_next = page_of(tile0 + BN);

  // queries: float32 from memory, split in two bfloat16 arrays (the first key tile is on its way meanwhile)
#pragma unroll 4
  for (int idx = tid; idx < BM * (D / 4); idx += NT) {
    const int i = idx / (D / 4), d = (idx - i * (D / 4)) * 4;
    const int pr = pr0 + i;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (pr < n_packed) {
      const int row = pr / G, hg = pr - row * G;
      v = *reinterpret_cast<const float4*>(q + ((size_t)(qs + row) * H + kvh * G + hg) * D + d);
    }
    uint2 h2, l2;
    split_pair(v.x, v.y, h2.x, l2.x);
    split_pair(v.z, v.w, h2.y, l2.y);
    *reinterpret_cast<uint2*>(Qh + i * LDQ + d) = h2;
    *reinterpret_cast<uint2*>(Ql + i * LDQ + d) = l2;
  }

  // this thread's two rows (g and g + 8 of the warp's sixteen): position, head, visible key range
  // rows mode: warp w owns rows 16 (w & 3) .. and the half w >> 2 of every key tile; keys mode: all
  // warps own rows 0 .. 15 and warp w < BN / 16 takes keys 16 w .. 16 w + 15 of every key tile
  const int row0 = keys_mode ? 0 : (warp & 3) * 16;
  const int koff = keys_mode ? warp * 16 : (warp >> 2) * (BN / 2);     // this warp's first key inside a tile
  const int kwidth = keys_mode ? 16 : BN / 2;
  const int n2_mine = keys_mode ? 1 : N2L;                              // its 16-key steps
  const bool idle_warp = koff >= BN;                                    // keys mode: more warps than 16-key parts
  int pos[2], head[2], lo[2], hi[2];
  bool valid[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int pr = pr0 + row0 + g + 8 * i;
    valid[i] = pr < n_packed;
    const int row = valid[i] ? pr / G : 0;
    pos[i] = pos0 + row;
    head[i] = kvh * G + (valid[i] ? pr - row * G : 0);
    lo[i] = valid[i] ? max(first_visible(pos[i], x.mask_kind, p.window), k_begin) : 1;
    hi[i] = valid[i] ? min(pos[i], k_end - 1) : 0;
  }
  // the keys any row of this warp sees: tiles outside are skipped by the warp
  const int warp_lo = __reduce_min_sync(0xffffffffu, min(valid[0] ? lo[0] : INT_MAX, valid[1] ? lo[1] : INT_MAX));
  const int warp_hi = __reduce_max_sync(0xffffffffu, max(valid[0] ? hi[0] : -1, valid[1] ? hi[1] : -1));
  // the keys EVERY row of this warp sees (empty when a row is idle): a tile inside needs no masking
  const bool all_valid = __all_sync(0xffffffffu, valid[0] && valid[1]);
  const int all_lo = all_valid ? __reduce_max_sync(0xffffffffu, max(lo[0], lo[1])) : INT_MAX;
  const int all_hi = all_valid ? __reduce_min_sync(0xffffffffu, min(hi[0], hi[1])) : -1;
  const float* bias_row[2] = {nullptr, nullptr};
  if (x.bias) {
    bias_row[0] = x.bias + (size_t)head[0] * x.bias_rows;
    bias_row[1] = x.bias + (size_t)head[1] * x.bias_rows;
  }

  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  float O[ONT][4];
#pragma unroll
  for (int on = 0; on < ONT; ++on) O[on][0] = O[on][1] = O[on][2] = O[on][3] = 0.f;

  int stage = 0;
  for (int ts = tile0; ts < k_end; ts += BN, stage ^= 1) {
    if (ts + BN < k_end) {
      load_tile(stage ^ 1, ts + BN, page_next);
      cp_async_commit();
      page_next = page_of(ts + 2 * BN);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();      // the tile has landed for every thread (and the queries are written, first time)
    const int tk = ts + koff;                 // this warp's first key of the tile
    const bool mine = !idle_warp && tk <= warp_hi && tk + kwidth > warp_lo;
    if (mine) {
      const bf16* Ks = KVs + stage * STAGE_ELEMS;
      const bf16* Vs = Ks + BN * LDK;
      float S[SNT][4];
#pragma unroll
      for (int nt = 0; nt < SNT; ++nt) S[nt][0] = S[nt][1] = S[nt][2] = S[nt][3] = 0.f;
      // the biases are requested before the products, which hide their latency; a distance outside
      // the table (a key no row sees) reads its nearest row and is masked below
      float B[SNT][4];
      if (x.bias) {
        const int last = x.bias_rows - 1;
        const int d0 = pos[0] - tk - 2 * t, d1 = pos[1] - tk - 2 * t;
#pragma unroll
        for (int nt = 0; nt < SNT; ++nt) {
          if ((nt >> 1) >= n2_mine) continue;
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            const int d = ((c >> 1) ? d1 : d0) - (nt * 8 + (c & 1));
            B[nt][c] = __ldg(bias_row[c >> 1] + min(max(d, 0), last));
          }
        }
      }
#pragma unroll
      for (int ks = 0; ks < KSTEPS; ++ks) {
        unsigned ah[4], al[4];
        const int qoff = (row0 + (lane & 7) + ((lane >> 3) & 1) * 8) * LDQ + ks * 16 + (lane >> 4) * 8;
        ldmatrix_x4(ah, Qh + qoff);
        ldmatrix_x4(al, Ql + qoff);
#pragma unroll
        for (int n2 = 0; n2 < N2L; ++n2) {
          if (n2 >= n2_mine) continue;
          unsigned kb[4];
          ldmatrix_x4(kb, Ks + (koff + (n2 * 2 + (lane >> 4)) * 8 + (lane & 7)) * LDK + ks * 16 + ((lane >> 3) & 1) * 8);
          mma_bf16(S[2 * n2], ah, kb[0], kb[1]);
          mma_bf16(S[2 * n2 + 1], ah, kb[2], kb[3]);
          mma_bf16(S[2 * n2], al, kb[0], kb[1]);
          mma_bf16(S[2 * n2 + 1], al, kb[2], kb[3]);
        }
      }
      // scale, bias, mask; the tile's row maxima
      float mx[2] = {-INFINITY, -INFINITY};
      if (!keys_mode && tk >= all_lo && tk + kwidth - 1 <= all_hi) {
        // every row of the warp sees every key of its part of the tile
#pragma unroll
        for (int nt = 0; nt < SNT; ++nt) {
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            const float sc = x.bias ? fmaf(S[nt][c], p.scale, B[nt][c]) : S[nt][c] * p.scale;
            S[nt][c] = sc;
            mx[c >> 1] = fmaxf(mx[c >> 1], sc);
          }
        }
      } else {
#pragma unroll
        for (int nt = 0; nt < SNT; ++nt) {
          const bool skip = (nt >> 1) >= n2_mine;
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            const int i = c >> 1;
            const int key = tk + nt * 8 + 2 * t + (c & 1);
            float sc = -INFINITY;
            if (!skip && key >= lo[i] && key <= hi[i])
              sc = x.bias ? fmaf(S[nt][c], p.scale, B[nt][c]) : S[nt][c] * p.scale;
            S[nt][c] = sc;
            mx[i] = fmaxf(mx[i], sc);
          }
        }
      }
      float m_safe[2];
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 1));
        mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 2));
        const float m_new = fmaxf(m_run[i], mx[i]);
        m_safe[i] = m_new == -INFINITY ? 0.f : m_new;
        const float alpha = __expf(m_run[i] - m_safe[i]);      // 0 while nothing was visible before
        m_run[i] = m_new;
        l_run[i] *= alpha;
#pragma unroll
        for (int on = 0; on < ONT; ++on) {
          O[on][2 * i] *= alpha;
          O[on][2 * i + 1] *= alpha;
        }
      }
#pragma unroll
      for (int nt = 0; nt < SNT; ++nt) {
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const float w = __expf(S[nt][c] - m_safe[c >> 1]);    // 0 for a masked score
          S[nt][c] = w;
          l_run[c >> 1] += w;
        }
      }
      // weights (two bfloat16 each) times values
#pragma unroll
      for (int kk = 0; kk < N2L; ++kk) {
        if (kk >= n2_mine) continue;
        unsigned ph[4], pl[4];
        split_pair(S[2 * kk][0], S[2 * kk][1], ph[0], pl[0]);
        split_pair(S[2 * kk][2], S[2 * kk][3], ph[1], pl[1]);
        split_pair(S[2 * kk + 1][0], S[2 * kk + 1][1], ph[2], pl[2]);
        split_pair(S[2 * kk + 1][2], S[2 * kk + 1][3], ph[3], pl[3]);
#pragma unroll
        for (int o2 = 0; o2 < ONT / 2; ++o2) {
          unsigned vb[4];
          ldmatrix_x4_trans(vb, Vs + (koff + kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * LDV + o2 * 16 + (lane >> 4) * 8);
          mma_bf16(O[2 * o2], ph, vb[0], vb[1]);
          mma_bf16(O[2 * o2 + 1], ph, vb[2], vb[3]);
          mma_bf16(O[2 * o2], pl, vb[0], vb[1]);
          mma_bf16(O[2 * o2 + 1], pl, vb[2], vb[3]);
        }
      }
    }
    __syncthreads();      // the stage is free for the fetch after the next
  }

  // a row's sum is spread over the four threads that hold its columns
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    l_run[i] += __shfl_xor_sync(0xffffffffu, l_run[i], 1);
    l_run[i] += __shfl_xor_sync(0xffffffffu, l_run[i], 2);
  }
  {
    // warps that saw different keys of the same rows are put together: in rows mode warp w + 4
    // hands its sums to warp w (slot w), in keys mode warps 1 .. 3 hand theirs to warp 0 (slots 0 .. 2)
    float* M = reinterpret_cast<float*>(KVs);
    const bool writer = !idle_warp && (keys_mode ? warp > 0 : warp >= 4);
    const int slot = keys_mode ? warp - 1 : (warp & 3);
    if (writer) {
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        float* dst = M + (size_t)(slot * 16 + g + 8 * i) * (E + 2);
#pragma unroll
        for (int on = 0; on < ONT; ++on)
          *reinterpret_cast<float2*>(dst + on * 8 + 2 * t) = make_float2(O[on][2 * i], O[on][2 * i + 1]);
        if (t == 0) {
          dst[E] = m_run[i];
          dst[E + 1] = l_run[i];
        }
      }
    }
    __syncthreads();
    if (writer || idle_warp) return;
    const int first_slot = keys_mode ? 0 : warp;
    const int n_slots = keys_mode ? min(4, BN / 16) - 1 : 1;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      float m = m_run[i];
      for (int w = 0; w < n_slots; ++w) m = fmaxf(m, M[(size_t)((first_slot + w) * 16 + g + 8 * i) * (E + 2) + E]);
      const float m_safe = m == -INFINITY ? 0.f : m;
      const float f0 = __expf(m_run[i] - m_safe);
      l_run[i] *= f0;
#pragma unroll
      for (int on = 0; on < ONT; ++on) {
        O[on][2 * i] *= f0;
        O[on][2 * i + 1] *= f0;
      }
      for (int w = 0; w < n_slots; ++w) {
        const float* src = M + (size_t)((first_slot + w) * 16 + g + 8 * i) * (E + 2);
        const float f = __expf(src[E] - m_safe);
        l_run[i] += src[E + 1] * f;
#pragma unroll
        for (int on = 0; on < ONT; ++on) {
          const float2 o = *reinterpret_cast<const float2*>(src + on * 8 + 2 * t);
          O[on][2 * i] += o.x * f;
          O[on][2 * i + 1] += o.y * f;
        }
      }
      m_run[i] = m;
    }
  }

#pragma unroll
  for (int i = 0; i < 2; ++i) {
    if (!valid[i]) continue;
    const int tok = qs + (pos[i] - pos0);
    if (nsplit <= 1) {
      float m = m_run[i], l = l_run[i], rescale = 1.f;
      if (x.unit_sink) add_unit_sink(m, l, rescale);
      const float inv = l > 0.f ? rescale / l : 0.f;
      bf16* o = (bf16*)p.out + ((size_t)tok * H + head[i]) * E;
      const bf16* gt = x.gate ? (const bf16*)x.gate + (size_t)tok * x.ldg + head[i] * E : nullptr;
      // the row's gate values are all requested before the first store (a store could alias them
      // for all the compiler knows, and each request would wait behind it); pairs where the gate's
      // rows start on 4-byte boundaries
      float2 gv[ONT];
      if (gt) {
        if (x.gate_pairs) {
#pragma unroll
          for (int on = 0; on < ONT; ++on)
            gv[on] = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(gt + on * 8 + 2 * t));
        } else {
#pragma unroll
          for (int on = 0; on < ONT; ++on)
            gv[on] = make_float2(__bfloat162float(gt[on * 8 + 2 * t]), __bfloat162float(gt[on * 8 + 2 * t + 1]));
        }
      }
#pragma unroll
      for (int on = 0; on < ONT; ++on) {
        const int e = on * 8 + 2 * t;
        float y0 = O[on][2 * i] * inv, y1 = O[on][2 * i + 1] * inv;
        if (gt) {
          y0 *= sigmoidf_(gv[on].x);
          y1 *= sigmoidf_(gv[on].y);
        }
        *reinterpret_cast<__nv_bfloat162*>(o + e) = __floats2bfloat162_rn(y0, y1);
      }
    } else {
      const int srow = p.tok_split_row[tok];
      const size_t b = ((size_t)srow * H + head[i]) * p.max_splits + split;
      float* po = p.part_o + b * E;
#pragma unroll
      for (int on = 0; on < ONT; ++on)
        *reinterpret_cast<float2*>(po + on * 8 + 2 * t) = make_float2(O[on][2 * i], O[on][2 * i + 1]);
      if (t == 0) {
        p.part_ml[b * 2] = m_run[i];
        p.part_ml[b * 2 + 1] = l_run[i];
      }
    }
  }
}
}  // namespace

PBE_EXPORT int pbe_masked_attention_mma_tile_rows() { return BM; }
PBE_EXPORT int pbe_masked_attention_mma_key_tile() { return BN; }

PBE_EXPORT int pbe_masked_attention_mma(const AttnParams* params, const float* bias, int bias_rows, int mask_kind,
                                        int unit_sink, const void* gate, int ldg, int num_work,
                                        cudaStream_t stream) {
  if (num_work <= 0) return 0;
  AttnParams p = *params;
  if (p.num_heads % p.num_kv_heads != 0 || p.tile_rows != BM || p.split_keys % BN != 0 || mask_kind < 0 ||
      mask_kind > 2 || (mask_kind != 0 && p.window < 1) || (bias && bias_rows < 1))
    return (int)cudaErrorInvalidValue;
  // rows are fetched in 16-byte pieces
  if ((((uintptr_t)p.q | (uintptr_t)p.k_cache | (uintptr_t)p.v_cache | (uintptr_t)p.part_o) & 15) != 0 ||
      ((uintptr_t)p.out & 3) != 0)
    return (int)cudaErrorMisalignedAddress;
  static bool opted = false;
  if (!opted && SMEM_BYTES > 48 * 1024) {
    const cudaError_t e = cudaFuncSetAttribute(masked_attention_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                               (int)SMEM_BYTES);
    if (e != cudaSuccess) return (int)e;
    opted = true;
  }
  MaskedExtra x{bias, bias_rows, mask_kind, unit_sink, gate, ldg, D, E};
  x.gate_pairs = gate != nullptr && ((uintptr_t)gate & 3) == 0 && (ldg & 1) == 0;
  launch_k(masked_attention_mma_kernel, dim3(num_work, p.num_kv_heads), NT, SMEM_BYTES, stream, p, x);
  return launch_status();
}
