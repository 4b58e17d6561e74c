// Attention over a compressed latent: every token keeps one row [c | kr] in the paged cache (c: a
// normed latent of `rank` values from which all heads' keys and values are linear maps; kr: one
// rotated key part of `rot` values that all heads share).  Keys and values are never expanded:
// the heads' key maps are applied to the queries instead and the heads' value maps to the
// attention's output,
//   score_h(i, j) = ((U_k,h^T q_h,i) . c_j + rope(q'_h,i) . kr_j) * scale,
//   out_h(i) = U_v,h (sum_j w_h(i, j) c_j),
// so that attention runs with one shared "key" row of rank + rot values and the first rank of
// them as the "value".  The softmax may have a sink: a learned logit per head in the denominator
// that has no key and no value.  Scores, weights and sums are float32.
//
//   latent_prepare   per token: RMS norms of the query latent and of c, rotation of kr, cache write
//   head_product     out[t, h, :] = W_h a[t, h, :] per head (the absorbed queries; the values with
//                    their sigmoid gate), float32 sums in a fixed order; optionally the rotated
//                    query part is appended
//   latent_attention causal attention of every row over its request's pages (same work list, row
//                    packing and key splits as the engine's other paged attention kernels)
//   latent_merge     the key splits' partial results and the sink into one result
#include "attention_params.cuh"
#include "common.cuh"
#include "pdl.cuh"

using namespace pbe;

namespace {
// ------------------------------------------------------------------------------------------------
struct PrepareParams {
  const void* proj;          // [T, ld]: the fused down projection
  int ld;
  int q_off, q_rank;         // columns of the query latent (q_rank 0: none)
  int c_off, rank;           // columns of the key/value latent
  int r_off, rot;            // columns of the shared rotated key part
  const float* q_gain;       // [q_rank]
  const float* c_gain;       // [rank]
  const float* inv_freq;     // [rot_dims / 2]
  int rot_dims;              // leading values of kr that are rotated, pairs (2i, 2i + 1)
  float rot_scale;           // cos and sin are both multiplied by it (1: a pure rotation)
  const int32_t* positions;  // [T]
  const int32_t* slots;      // [T] page * page_tokens + offset, negative: nothing is written
  void* q_lat;               // [T, q_rank] normed query latent
  void* cache;               // [pages * page_tokens, rank + rot] or null
  float eps;
};

template <typename T>
__global__ void latent_prepare_kernel(PrepareParams p) {
  __shared__ float red[33];
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const T* row = (const T*)p.proj + (size_t)t * p.ld;
  if (p.q_rank > 0) {
    float ss = 0.f;
    for (int i = threadIdx.x; i < p.q_rank; i += blockDim.x) {
      const float v = to_float(row[p.q_off + i]);
      ss += v * v;
    }
    const float scale = rsqrtf(block_sum(ss, red) / (float)p.q_rank + p.eps);
    T* o = (T*)p.q_lat + (size_t)t * p.q_rank;
    for (int i = threadIdx.x; i < p.q_rank; i += blockDim.x)
      o[i] = from_float<T>((p.q_gain[i] * to_float(row[p.q_off + i])) * scale);
  }
  const int slot = p.slots ? p.slots[t] : -1;
  if (p.cache == nullptr || slot < 0) return;
  T* dst = (T*)p.cache + (size_t)slot * (p.rank + p.rot);
  float ss = 0.f;
  for (int i = threadIdx.x; i < p.rank; i += blockDim.x) {
    const float v = to_float(row[p.c_off + i]);
    ss += v * v;
  }
  const float scale = rsqrtf(block_sum(ss, red) / (float)p.rank + p.eps);
  for (int i = threadIdx.x; i < p.rank; i += blockDim.x)
    dst[i] = from_float<T>((p.c_gain[i] * to_float(row[p.c_off + i])) * scale);
  const float pos = (float)p.positions[t];
  for (int i = threadIdx.x; i < p.rot / 2; i += blockDim.x) {
    const float u = to_float(row[p.r_off + 2 * i]), v = to_float(row[p.r_off + 2 * i + 1]);
    float a = u, b = v;
    if (2 * i + 1 < p.rot_dims) {
      float sn, cs;
      sincosf(pos * p.inv_freq[i], &sn, &cs);
      sn *= p.rot_scale;
      cs *= p.rot_scale;
      a = u * cs - v * sn;
      b = v * cs + u * sn;
    }
    dst[p.rank + 2 * i] = from_float<T>(a);
    dst[p.rank + 2 * i + 1] = from_float<T>(b);
  }
  if ((p.rot & 1) && threadIdx.x == 0) dst[p.rank + p.rot - 1] = row[p.r_off + p.rot - 1];
}

// ------------------------------------------------------------------------------------------------
// out[t, h, n] = sum_k a[t, h, k] * w[h][k * wk + n * wn]  for n < N, per head h
struct HeadProductParams {
  const void* a;             // element (row 0, head 0, 0); row stride lda, head stride ha
  int lda, ha;
  const void* w;             // head stride hw; element strides wk (along k) and wn (along n)
  long long hw;
  int wk, wn;
  void* out;                 // row stride ldo, head stride ho
  int ldo, ho;
  int T, H, K, N;
  // optional tail: out[t, h, N + i] = rope(a[t, h, K + i]) for i < rot (pairs (2i, 2i+1) of the first rot_dims)
  int rot, rot_dims;
  const float* inv_freq;
  const int32_t* positions;
  // optional gate: the result is multiplied by sigmoid(gate[t * ldg + h]), or (gate_each) by
  // sigmoid(gate[t * ldg + h * N + n]), a gate per output value; the gate has the weights' dtype
  const void* gate;
  int ldg;
  float rot_scale;           // cos and sin of the tail's rotation are both multiplied by it
  int gate_each;
};

constexpr int HP_TM = 16, HP_TN = 64, HP_TK = 32;

template <typename TA, typename TW, typename TO>
__global__ void __launch_bounds__(256) head_product_kernel(HeadProductParams p) {
  __shared__ float As[HP_TM][HP_TK + 1];
  __shared__ float Ws[HP_TK][HP_TN + 1];
  pdl_launch_dependents();
  pdl_wait();
  const int h = blockIdx.y;
  const int t0 = blockIdx.x * HP_TM;
  const int n0 = blockIdx.z * HP_TN;
  const int tid = threadIdx.x;
  const int tn = tid % HP_TN, tg = tid / HP_TN;           // column, and which four rows
  const TA* a = (const TA*)p.a + (size_t)h * p.ha;
  const TW* w = (const TW*)p.w + (size_t)h * p.hw;
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  for (int k0 = 0; k0 < p.K; k0 += HP_TK) {
    for (int idx = tid; idx < HP_TM * HP_TK; idx += 256) {
      const int i = idx / HP_TK, k = idx - i * HP_TK;
      const int t = t0 + i;
      As[i][k] = (t < p.T && k0 + k < p.K) ? to_float(a[(size_t)t * p.lda + k0 + k]) : 0.f;
    }
    for (int idx = tid; idx < HP_TK * HP_TN; idx += 256) {
      // the faster-running index follows the operand's unit stride
      int k, n;
      if (p.wn == 1) { k = idx / HP_TN; n = idx - k * HP_TN; } else { n = idx / HP_TK; k = idx - n * HP_TK; }
      Ws[k][n] = (k0 + k < p.K && n0 + n < p.N) ? to_float(w[(size_t)(k0 + k) * p.wk + (size_t)(n0 + n) * p.wn]) : 0.f;
    }
    __syncthreads();
#pragma unroll 8
    for (int k = 0; k < HP_TK; ++k) {
      const float wv = Ws[k][tn];
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[j] = fmaf(As[tg * 4 + j][k], wv, acc[j]);
    }
    __syncthreads();
  }
  const int n = n0 + tn;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int t = t0 + tg * 4 + j;
    if (t >= p.T || n >= p.N) continue;
    float v = acc[j];
    if (p.gate) {
      const float g = to_float(((const TW*)p.gate)[(size_t)t * p.ldg + (p.gate_each ? (size_t)h * p.N + n : (size_t)h)]);
      v *= 1.0f / (1.0f + expf(-g));
    }
    ((TO*)p.out)[(size_t)t * p.ldo + (size_t)h * p.ho + n] = from_float<TO>(v);
  }
  if (p.rot > 0 && blockIdx.z == 0) {
    for (int idx = tid; idx < HP_TM * (p.rot / 2); idx += 256) {
      const int i = idx / (p.rot / 2), pr = idx - i * (p.rot / 2);
      const int t = t0 + i;
      if (t >= p.T) continue;
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
      TO* dst = (TO*)p.out + (size_t)t * p.ldo + (size_t)h * p.ho + p.N;
      dst[2 * pr] = from_float<TO>(x);
      dst[2 * pr + 1] = from_float<TO>(y);
    }
  }
}

// ------------------------------------------------------------------------------------------------
struct LatentAttnParams {
  AttnParams a;              // q: float32 [T, H, dk]; k_cache: [page][page_tokens][dk]; out: float32 [T, H, dv];
                             // num_kv_heads 1, tile_rows a multiple of 16
  const float* sink;         // [H] or null
  int dk, dv;                // width of a cache row; its leading dv values are the value
  int sub;                   // blocks (along z) that share a key split of a split row, each an equal part of
                             // its keys and a partial result of its own: slot split * sub + z of max_splits * sub
};

constexpr int LA_BM = 16;    // packed rows (row x head) a block
constexpr int LA_BN = 32;    // keys a tile, one per lane
constexpr int LA_WARPS = 4;
constexpr int LA_RPW = LA_BM / LA_WARPS;

template <typename T, int DPL>
__global__ void __launch_bounds__(LA_WARPS * 32) latent_attention_kernel(LatentAttnParams lp) {
  extern __shared__ __align__(16) float smem[];
  const AttnParams& p = lp.a;
  const int DK = lp.dk, DV = lp.dv;
  const int KS = DK | 1;                 // odd row stride: a key per lane without bank conflicts
  float* Qs = smem;                      // [LA_BM][DK]
  float* Ks = Qs + LA_BM * DK;           // [LA_BN][KS]
  pdl_launch_dependents();
  pdl_wait();
  const int32_t* work = p.work + (size_t)blockIdx.x * 4;
  const int r = work[0];
  if (r < 0) return;
  const int split = work[2], nsplit = work[3];
  const int H = p.num_heads, G = H, P = p.page_tokens;
  const int qs = p.q_start[r], nq = p.q_len[r], sl = p.seq_len[r];
  const int n_packed = nq * G;
  const int pr0 = work[1] * p.tile_rows + blockIdx.y * LA_BM;
  if (pr0 >= n_packed || blockIdx.y * LA_BM >= p.tile_rows) return;
  const int row_lo = pr0 / G;
  const int row_hi = (min(n_packed, pr0 + LA_BM) - 1) / G;
  const int pos0 = sl - nq;
  const int hi_key = pos0 + row_hi + 1;
  const int lo_key = p.window > 0 ? max(0, pos0 + row_lo - p.window + 1) : 0;
  int k_begin = lo_key, k_end = hi_key;
  if (nsplit > 1) {
    const int lo_req = p.window > 0 ? max(0, pos0 - p.window + 1) : 0;
    const int s0 = lo_req / p.split_keys;
    k_begin = max(lo_key, (s0 + split) * p.split_keys);
    k_end = min(hi_key, (s0 + split + 1) * p.split_keys);
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const float* q = (const float*)p.q;
  const T* kc = (const T*)p.k_cache;
  const int32_t* bt = p.block_table + (size_t)r * p.bt_stride;

  for (int idx = threadIdx.x; idx < LA_BM * DK; idx += blockDim.x) {
    const int i = idx / DK, d = idx - i * DK;
    const int pr = pr0 + i;
    float v = 0.f;
    if (pr < n_packed) {
      const int row = pr / G, hg = pr - row * G;
      v = q[((size_t)(qs + row) * H + hg) * DK + d];
    }
    Qs[idx] = v;
  }
  float m_run[LA_RPW], l_run[LA_RPW], acc[LA_RPW][DPL];
#pragma unroll
  for (int j = 0; j < LA_RPW; ++j) {
    m_run[j] = -INFINITY;
    l_run[j] = 0.f;
#pragma unroll
    for (int i = 0; i < DPL; ++i) acc[j][i] = 0.f;
  }
  const int tile0 = (k_begin / LA_BN) * LA_BN;
  for (int ts = tile0; ts < k_end; ts += LA_BN) {
    __syncthreads();       // the tile before is consumed (and Qs is written, the first time)
    // every warp brings eight of the tile's rows, the lanes along a row
    {
      const int my_key = ts + lane;
      int my_page = -1;
      if (my_key >= k_begin && my_key < k_end) my_page = bt[my_key / P];
#pragma unroll
      for (int jj = 0; jj < LA_BN / LA_WARPS; ++jj) {
        const int j = warp + jj * LA_WARPS;
        const int key = ts + j;
        const int page = __shfl_sync(0xffffffffu, my_page, j);
        float* dst = Ks + j * KS;
        if (page >= 0) {
          const T* src = kc + ((size_t)page * P + (key % P)) * DK;
          for (int d = lane; d < DK; d += 32) dst[d] = to_float(src[d]);
        } else {
          for (int d = lane; d < DK; d += 32) dst[d] = 0.f;
        }
      }
    }
    __syncthreads();
    float s[LA_RPW];
#pragma unroll
    for (int j = 0; j < LA_RPW; ++j) s[j] = 0.f;
    {
      const float* krow = Ks + lane * KS;
      for (int d = 0; d < DK; ++d) {
        const float kv = krow[d];
#pragma unroll
        for (int j = 0; j < LA_RPW; ++j) s[j] = fmaf(Qs[(warp + j * LA_WARPS) * DK + d], kv, s[j]);
      }
    }
    float pj[LA_RPW];
#pragma unroll
    for (int j = 0; j < LA_RPW; ++j) {
      const int pr = pr0 + warp + j * LA_WARPS;
      pj[j] = 0.f;
      if (pr >= n_packed) continue;
      const int pos = pos0 + pr / G;
      const int key = ts + lane;
      const int row_lo_key = p.window > 0 ? pos - p.window + 1 : 0;
      const bool visible = key >= k_begin && key < k_end && key <= pos && key >= row_lo_key;
      const float sc = visible ? s[j] * p.scale : -INFINITY;
      const float m_new = fmaxf(m_run[j], warp_max(sc));
      if (m_new == -INFINITY) continue;
      pj[j] = visible ? expf(sc - m_new) : 0.f;
      const float alpha = expf(m_run[j] - m_new);
      l_run[j] = l_run[j] * alpha + warp_sum(pj[j]);
      m_run[j] = m_new;
#pragma unroll
      for (int ii = 0; ii < DPL; ++ii) acc[j][ii] *= alpha;
    }
    for (int kk = 0; kk < LA_BN; ++kk) {
      float vv[DPL];
#pragma unroll
      for (int ii = 0; ii < DPL; ++ii) {
        const int d = lane + ii * 32;
        vv[ii] = d < DV ? Ks[kk * KS + d] : 0.f;
      }
#pragma unroll
      for (int j = 0; j < LA_RPW; ++j) {
        const float pk = __shfl_sync(0xffffffffu, pj[j], kk);
#pragma unroll
        for (int ii = 0; ii < DPL; ++ii) acc[j][ii] = fmaf(pk, vv[ii], acc[j][ii]);
      }
    }
  }
#pragma unroll
  for (int j = 0; j < LA_RPW; ++j) {
    const int pr = pr0 + warp + j * LA_WARPS;
    if (pr >= n_packed) continue;
    const int row = pr / G, head = pr - row * G;
    const int t = qs + row;
    if (nsplit <= 1) {
      // the sink joins the denominator once: a logit without key or value
      float m_fin = m_run[j], l = l_run[j], factor = 1.f;
      if (lp.sink) {
        const float sk = lp.sink[head];
        m_fin = fmaxf(m_run[j], sk);
        factor = expf(m_run[j] - m_fin);
        l = l * factor + expf(sk - m_fin);
      }
      const float inv = l > 0.f ? factor / l : 0.f;
      float* o = (float*)p.out + ((size_t)t * H + head) * DV;
#pragma unroll
      for (int ii = 0; ii < DPL; ++ii) {
        const int d = lane + ii * 32;
        if (d < DV) o[d] = acc[j][ii] * inv;
      }
    } else {
      const int srow = p.tok_split_row[t];
      const size_t base = ((size_t)srow * H + head) * p.max_splits + split;
      float* po = p.part_o + base * DV;
#pragma unroll
      for (int ii = 0; ii < DPL; ++ii) {
        const int d = lane + ii * 32;
        if (d < DV) po[d] = acc[j][ii];
      }
      if (lane == 0) {
        p.part_ml[base * 2] = m_run[j];
        p.part_ml[base * 2 + 1] = l_run[j];
      }
    }
  }
}

// ------------------------------------------------------------------------------------------------
// The same attention on the tensor cores (mma.sync m16n8k16, bfloat16 operands, float32 sums) for
// bfloat16 caches whose rows are a multiple of 16 values wide.  Four warps take 16 packed rows and
// tiles of 32 keys; a block is RG such groups of four warps (16 RG rows) that share every key tile,
// so the tile crosses from the L2 cache once for all of them: one group for decoded tokens, four for
// prompt portions.  The queries are rounded to bfloat16 once (operands of a product, as the
// cached rows are); scores, maxima, sums and weights are float32.  Per tile: warp w multiplies the
// queries with keys 8w .. 8w+7, the score blocks meet in shared memory, every warp takes the softmax
// step of the whole tile for its rows, and multiplies the weights with its own quarter of the value
// columns.  A weight enters that product as the sum of two bfloat16 numbers (its rounding and the
// rounding of what is left), so it keeps 16 bits of mantissa, not 8.
__device__ __forceinline__ void mma_bf16(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const unsigned*>(&v);
}

constexpr int LM_BN = 32;      // keys a tile
constexpr int LM_WARPS = 4;

// NT: tiles of 8 value columns a warp owns (four warps cover 32 * NT >= dv columns); RG: row groups
template <int NT, int RG>
__global__ void __launch_bounds__(LM_WARPS * 32 * RG) latent_attention_mma_kernel(LatentAttnParams lp) {
  constexpr int ROWS = LA_BM * RG;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const AttnParams& p = lp.a;
  const int DK = lp.dk, DV = lp.dv;
  const int QSTR = DK + 8;                                   // bfloat16 elements a row of Qs
  const int wide = max(DK, 32 * NT);
  const int KSTR = wide + 8;                                 // and of Ks: rows stay 16-byte aligned, banks shift
  __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(smem_raw);                 // [ROWS][QSTR]
  __nv_bfloat16* Kbuf = Qs + ROWS * QSTR;                                          // [2][LM_BN][KSTR]
  float* Ss = reinterpret_cast<float*>(Kbuf + 2 * LM_BN * KSTR);                   // [ROWS][LM_BN + 1]
  pdl_launch_dependents();
  pdl_wait();
  const int32_t* work = p.work + (size_t)blockIdx.x * 4;
  const int r = work[0];
  if (r < 0) return;
  const int split = work[2], nsplit = work[3];
  const int H = p.num_heads, G = H, P = p.page_tokens;
  const int qs = p.q_start[r], nq = p.q_len[r], sl = p.seq_len[r];
  const int n_packed = nq * G;
  const int pr0 = work[1] * p.tile_rows + blockIdx.y * ROWS;
  if (pr0 >= n_packed || blockIdx.y * ROWS >= p.tile_rows) return;
  const int row_lo = pr0 / G;
  const int row_hi = (min(n_packed, pr0 + ROWS) - 1) / G;
  const int pos0 = sl - nq;
  const int hi_key = pos0 + row_hi + 1;
  const int lo_key = p.window > 0 ? max(0, pos0 + row_lo - p.window + 1) : 0;
  int k_begin = lo_key, k_end = hi_key;
  const int Z = lp.sub, z = blockIdx.z;
  if (nsplit > 1) {
    const int lo_req = p.window > 0 ? max(0, pos0 - p.window + 1) : 0;
    const int s0 = lo_req / p.split_keys;
    const int part = p.split_keys / Z;              // a multiple of the key tile (the launcher checks)
    k_begin = max(lo_key, (s0 + split) * p.split_keys + z * part);
    k_end = min(hi_key, (s0 + split) * p.split_keys + (z + 1) * part);
  } else if (z > 0) {
    return;
  }
  const int tid = threadIdx.x, lane = tid & 31;
  const int warp = (tid >> 5) & 3, rg = tid >> 7;            // the warp's place in its group of four, and the group
  const int g8 = lane >> 2, q2 = (lane & 3) * 2;             // the thread's rows g8 and g8 + 8 of the group, its column pair
  const float* q = (const float*)p.q;
  const __nv_bfloat16* kc = (const __nv_bfloat16*)p.k_cache;
  const int32_t* bt = p.block_table + (size_t)r * p.bt_stride;

  {
    // the queries: 16-byte loads, four of a thread's in flight at once, rounded as they are staged
    const int qchunks = DK / 4, total = ROWS * qchunks;
    for (int first = 0; first < total; first += (int)blockDim.x * 4) {
      float4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int idx = first + tid + u * (int)blockDim.x;
        v[u] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (idx < total) {
          const int i = idx / qchunks, c = idx - i * qchunks;
          const int pr = pr0 + i;
          if (pr < n_packed) {
            const int row = pr / G, hg = pr - row * G;
            v[u] = *reinterpret_cast<const float4*>(q + ((size_t)(qs + row) * H + hg) * DK + c * 4);
          }
        }
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int idx = first + tid + u * (int)blockDim.x;
        if (idx < total) {
          const int i = idx / qchunks, c = idx - i * qchunks;
          uint2 packed;
          packed.x = pack_bf16(v[u].x, v[u].y);
          packed.y = pack_bf16(v[u].z, v[u].w);
          *reinterpret_cast<uint2*>(Qs + i * QSTR + c * 4) = packed;
        }
      }
    }
  }
  // columns of the key tiles beyond the cached row (read as value columns that are never stored) stay zero
  for (int idx = tid; idx < 2 * LM_BN * (KSTR - DK); idx += blockDim.x) {
    const int j = idx / (KSTR - DK), d = DK + idx - j * (KSTR - DK);
    Kbuf[j * KSTR + d] = __float2bfloat16_rn(0.f);
  }
  float acc[NT][4];
#pragma unroll
  for (int i = 0; i < NT; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  int pos_row[2];                                              // the rows' positions, -1: no such row
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int pr = pr0 + rg * LA_BM + g8 + 8 * h;
    pos_row[h] = pr < n_packed ? pos0 + pr / G : -1;
  }
  const int chunks = DK / 8;                                  // 16-byte pieces of a cached row
  const int col0 = warp * NT * 8;                             // this warp's first value column
  const int tile0 = (k_begin / LM_BN) * LM_BN;
  // A tile's rows arrive by asynchronous 16-byte copies, four threads a row (its page is looked up
  // once), into the buffer that is not being multiplied: the tile after this one is on its way while
  // this one is worked on.
  auto fetch = [&](int buf, int ts) {
    constexpr int PER_ROW = 4 * RG;      // threads that share a row
    const int j = tid / PER_ROW, key = ts + j;
    int page = -1;
    if (key >= k_begin && key < k_end) page = bt[key / P];
    __nv_bfloat16* dst = Kbuf + ((size_t)buf * LM_BN + j) * KSTR;
    if (page >= 0) {
      const __nv_bfloat16* src = kc + ((size_t)page * P + (key % P)) * DK;
      for (int c = tid % PER_ROW; c < chunks; c += PER_ROW) {
        const unsigned to = (unsigned)__cvta_generic_to_shared(dst + c * 8);
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(to), "l"(src + c * 8) : "memory");
      }
    } else {
      for (int c = tid % PER_ROW; c < chunks; c += PER_ROW) *reinterpret_cast<uint4*>(dst + c * 8) = make_uint4(0u, 0u, 0u, 0u);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  if (tile0 < k_end) fetch(0, tile0);
  int buf = 0;
  for (int ts = tile0; ts < k_end; ts += LM_BN, buf ^= 1) {
    __syncthreads();       // the tile before is consumed (and Qs is written, the first time)
    const __nv_bfloat16* Ks = Kbuf + (size_t)buf * LM_BN * KSTR;
    if (ts + LM_BN < k_end) {
      fetch(buf ^ 1, ts + LM_BN);
      asm volatile("cp.async.wait_group 1;" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    __syncthreads();
    {
      // scores of the 16 rows against this warp's eight keys
      // two sums in turn, so that a product need not wait for the one before it; fragments by ldmatrix
      // (a 16 x 16 piece of the queries, an 8 x 16 piece of the keys, one instruction each)
      float c[4] = {0.f, 0.f, 0.f, 0.f}, c2[4] = {0.f, 0.f, 0.f, 0.f};
      const __nv_bfloat16* qa = Qs + (rg * LA_BM + (lane & 7) + ((lane >> 3) & 1) * 8) * QSTR + (lane >> 4) * 8;
      const __nv_bfloat16* kb = Ks + (warp * 8 + (lane & 7)) * KSTR + ((lane >> 3) & 1) * 8;
      auto step = [&](int kk, float (&sum)[4]) {
        unsigned a[4], b0, b1;
        const unsigned qaddr = (unsigned)__cvta_generic_to_shared(qa + kk);
        const unsigned kaddr = (unsigned)__cvta_generic_to_shared(kb + kk);
        asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                     : "=r"(a[0]), "=r"(a[1]), "=r"(a[2]), "=r"(a[3]) : "r"(qaddr));
        asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];" : "=r"(b0), "=r"(b1) : "r"(kaddr));
        mma_bf16(sum, a, b0, b1);
      };
      int kk = 0;
      for (; kk + 32 <= DK; kk += 32) {
        step(kk, c);
        step(kk + 16, c2);
      }
      if (kk < DK) step(kk, c);
#pragma unroll
      for (int i = 0; i < 4; ++i) c[i] += c2[i];
      float* s0 = Ss + (rg * LA_BM + g8) * (LM_BN + 1) + warp * 8 + q2;
      s0[0] = c[0]; s0[1] = c[1];
      s0[8 * (LM_BN + 1)] = c[2]; s0[8 * (LM_BN + 1) + 1] = c[3];
    }
    __syncthreads();
    // the softmax step of the whole tile for rows g8 and g8 + 8; this thread holds the weights of
    // keys q2, q2+1, q2+8, q2+9 (+16 for the tile's second half), as the products' A operand wants
    unsigned a_hi[2][4], a_lo[2][4];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const float* srow = Ss + (rg * LA_BM + g8 + 8 * h) * (LM_BN + 1);
      const int pos = pos_row[h];
      const int row_lo_key = p.window > 0 ? pos - p.window + 1 : 0;
      float sc[8];
      float mx = -INFINITY;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int col = (i >> 2) * 16 + ((i >> 1) & 1) * 8 + q2 + (i & 1);
        const int key = ts + col;
        const bool visible = pos >= 0 && key >= k_begin && key < k_end && key <= pos && key >= row_lo_key;
        sc[i] = visible ? srow[col] * p.scale : -INFINITY;
        mx = fmaxf(mx, sc[i]);
      }
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
      const float m_new = fmaxf(m_run[h], mx);
      float alpha = 1.f, sum = 0.f;
      float pw[8];
      if (m_new == -INFINITY) {
#pragma unroll
        for (int i = 0; i < 8; ++i) pw[i] = 0.f;
      } else {
        alpha = expf(m_run[h] - m_new);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          pw[i] = sc[i] == -INFINITY ? 0.f : expf(sc[i] - m_new);
          sum += pw[i];
        }
        m_run[h] = m_new;
      }
      sum += __shfl_xor_sync(0xffffffffu, sum, 1);
      sum += __shfl_xor_sync(0xffffffffu, sum, 2);
      l_run[h] = l_run[h] * alpha + sum;
#pragma unroll
      for (int i = 0; i < NT; ++i) { acc[i][2 * h] *= alpha; acc[i][2 * h + 1] *= alpha; }
      // pairs (i, i + 1): half j = i / 4 of the tile, register h (cols q2..) or h + 2 (cols q2 + 8..)
#pragma unroll
      for (int i = 0; i < 8; i += 2) {
        const float h0 = __bfloat162float(__float2bfloat16_rn(pw[i])), h1 = __bfloat162float(__float2bfloat16_rn(pw[i + 1]));
        const int j = i >> 2, reg = h + ((i >> 1) & 1) * 2;
        a_hi[j][reg] = pack_bf16(h0, h1);
        a_lo[j][reg] = pack_bf16(pw[i] - h0, pw[i + 1] - h1);
      }
    }
    // weighted values: this warp's columns, the value rows transposed as they are loaded
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const __nv_bfloat16* vrow = Ks + (16 * j + (lane & 15)) * KSTR + col0;
      // four column tiles at a time: their products with the weights' first terms, then with the
      // second terms, so that no product waits for the one issued just before it
      constexpr int GRP = NT < 4 ? NT : 4;
#pragma unroll
      for (int nt0 = 0; nt0 < NT; nt0 += GRP) {
        unsigned b[GRP][2];
#pragma unroll
        for (int u = 0; u < GRP; ++u) {
          const unsigned addr = (unsigned)__cvta_generic_to_shared(vrow + (nt0 + u) * 8);
          asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];"
                       : "=r"(b[u][0]), "=r"(b[u][1]) : "r"(addr));
        }
#pragma unroll
        for (int u = 0; u < GRP; ++u) mma_bf16(acc[nt0 + u], a_hi[j], b[u][0], b[u][1]);
#pragma unroll
        for (int u = 0; u < GRP; ++u) mma_bf16(acc[nt0 + u], a_lo[j], b[u][0], b[u][1]);
      }
    }
  }
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int pr = pr0 + rg * LA_BM + g8 + 8 * h;
    if (pr >= n_packed) continue;
    const int row = pr / G, head = pr - row * G;
    const int t = qs + row;
    if (nsplit <= 1) {
      float m_fin = m_run[h], l = l_run[h], factor = 1.f;
      if (lp.sink) {
        const float sk = lp.sink[head];
        m_fin = fmaxf(m_run[h], sk);
        factor = expf(m_run[h] - m_fin);
        l = l * factor + expf(sk - m_fin);
      }
      const float inv = l > 0.f ? factor / l : 0.f;
      float* o = (float*)p.out + ((size_t)t * H + head) * DV;
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        const int d = col0 + nt * 8 + q2;
        if (d < DV) o[d] = acc[nt][2 * h] * inv;
        if (d + 1 < DV) o[d + 1] = acc[nt][2 * h + 1] * inv;
      }
    } else {
      const int srow = p.tok_split_row[t];
      const size_t base = ((size_t)srow * H + head) * (p.max_splits * Z) + split * Z + z;
      float* po = p.part_o + base * DV;
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        const int d = col0 + nt * 8 + q2;
        if (d < DV) po[d] = acc[nt][2 * h];
        if (d + 1 < DV) po[d + 1] = acc[nt][2 * h + 1];
      }
      if (warp == 0 && (lane & 3) == 0) {
        p.part_ml[base * 2] = m_run[h];
        p.part_ml[base * 2 + 1] = l_run[h];
      }
    }
  }
}

template <int NT, int RG>
int launch_latent_mma(const LatentAttnParams& lp, int num_work, cudaStream_t stream) {
  constexpr int ROWS = LA_BM * RG;
  const int wide = lp.dk > 32 * NT ? lp.dk : 32 * NT;
  const size_t smem = 2 * ((size_t)ROWS * (lp.dk + 8) + 2 * (size_t)LM_BN * (wide + 8)) + sizeof(float) * ROWS * (LM_BN + 1);
  if (smem > 200 * 1024) return (int)cudaErrorInvalidValue;
  static size_t opted = 48 * 1024;
  if (smem > opted) {
    cudaFuncSetAttribute(latent_attention_mma_kernel<NT, RG>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    opted = 200 * 1024;
  }
  dim3 grid(num_work, (lp.a.tile_rows + ROWS - 1) / ROWS, lp.sub);
  launch_k(latent_attention_mma_kernel<NT, RG>, grid, LM_WARPS * 32 * RG, smem, stream, lp);
  return launch_status();
}

// wide_blocks: blocks of four row groups (prompt portions) when the work list's tiles hold 64 rows
int dispatch_latent_mma(const LatentAttnParams& lp, int num_work, bool wide_blocks, cudaStream_t stream) {
  const int nt = (lp.dv + 31) / 32;
  const size_t wide_smem = 2 * ((size_t)64 * (lp.dk + 8) + 2 * (size_t)LM_BN * ((lp.dk > 32 * nt ? lp.dk : 32 * nt) + 8)) +
                           sizeof(float) * 64 * (LM_BN + 1);
  const bool four = wide_blocks && lp.a.tile_rows % 64 == 0 && wide_smem <= 200 * 1024;
#define PBE_LM(N)                                                                                   \
  return four ? launch_latent_mma<N, 4>(lp, num_work, stream) : launch_latent_mma<N, 1>(lp, num_work, stream)
  if (nt <= 1) { PBE_LM(1); }
  if (nt <= 2) { PBE_LM(2); }
  if (nt <= 4) { PBE_LM(4); }
  if (nt <= 8) { PBE_LM(8); }
  if (nt <= 16) { PBE_LM(16); }
#undef PBE_LM
  return (int)cudaErrorInvalidValue;
}

struct LatentMergeParams {
  AttnMergeParams m;         // out: float32 [T, H, head_dim]; max_splits counts every partial slot of a row and head
  const float* sink;
  int sub;                   // partial results per key split
};

__global__ void latent_merge_kernel(LatentMergeParams lp) {
  extern __shared__ float weight[];        // [slots]: exp(m_s - m) of every partial result
  __shared__ float red[33];
  const AttnMergeParams& p = lp.m;
  pdl_launch_dependents();
  pdl_wait();
  const int srow = blockIdx.x, head = blockIdx.y;
  if (p.split_counts[srow] <= 1) return;
  const int n = p.split_counts[srow] * lp.sub;
  const int t = p.split_tokens[srow];
  const size_t base = ((size_t)srow * p.num_heads + head) * p.max_splits;
  // the partial results' maxima and sums are fetched side by side, one a thread
  float m_mine = -INFINITY;
  for (int s0 = threadIdx.x; s0 < n; s0 += blockDim.x) m_mine = fmaxf(m_mine, p.part_ml[(base + s0) * 2]);
  m_mine = warp_max(m_mine);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = m_mine;
  __syncthreads();
  float m = lp.sink ? lp.sink[head] : -INFINITY;
  for (int w = 0; w < (int)(blockDim.x >> 5); ++w) m = fmaxf(m, red[w]);
  float l_mine = 0.f;
  for (int s0 = threadIdx.x; s0 < n; s0 += blockDim.x) {
    const float ms = p.part_ml[(base + s0) * 2];
    const float w = ms == -INFINITY ? 0.f : expf(ms - m);
    weight[s0] = w;
    l_mine += w * p.part_ml[(base + s0) * 2 + 1];
  }
  const float l = block_sum(l_mine, red) + (lp.sink ? expf(lp.sink[head] - m) : 0.f);   // also publishes weight[]
  const float inv = l > 0.f ? 1.0f / l : 0.f;
  float* o = (float*)p.out + ((size_t)t * p.num_heads + head) * p.head_dim;
  const float* po = p.part_o + base * p.head_dim;
  for (int d = threadIdx.x; d < p.head_dim; d += blockDim.x) {
    float a[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    int s0 = 0;
    for (; s0 + 8 <= n; s0 += 8) {         // eight loads in flight; the order of the sum is fixed by n alone
      float v[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) v[u] = po[(size_t)(s0 + u) * p.head_dim + d];
#pragma unroll
      for (int u = 0; u < 8; ++u) a[u] = fmaf(v[u], weight[s0 + u], a[u]);
    }
    for (; s0 < n; ++s0) a[0] = fmaf(po[(size_t)s0 * p.head_dim + d], weight[s0], a[0]);
    o[d] = (((a[0] + a[1]) + (a[2] + a[3])) + ((a[4] + a[5]) + (a[6] + a[7]))) * inv;
  }
}

template <typename T, int DPL>
int launch_latent(const LatentAttnParams& lp, int num_work, cudaStream_t stream) {
  const size_t smem = sizeof(float) * ((size_t)LA_BM * lp.dk + (size_t)LA_BN * (lp.dk | 1));
  if (smem > 200 * 1024) return (int)cudaErrorInvalidValue;
  static size_t opted = 48 * 1024;
  if (smem > opted) {
    cudaFuncSetAttribute(latent_attention_kernel<T, DPL>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    opted = 200 * 1024;
  }
  dim3 grid(num_work, lp.a.tile_rows / LA_BM);
  launch_k(latent_attention_kernel<T, DPL>, grid, LA_WARPS * 32, smem, stream, lp);
  return launch_status();
}

template <typename T>
int dispatch_latent(const LatentAttnParams& lp, int num_work, cudaStream_t stream) {
  const int dpl = (lp.dv + 31) / 32;
  if (dpl <= 1) return launch_latent<T, 1>(lp, num_work, stream);
  if (dpl <= 2) return launch_latent<T, 2>(lp, num_work, stream);
  if (dpl <= 4) return launch_latent<T, 4>(lp, num_work, stream);
  if (dpl <= 8) return launch_latent<T, 8>(lp, num_work, stream);
  if (dpl <= 16) return launch_latent<T, 16>(lp, num_work, stream);
  return (int)cudaErrorInvalidValue;
}
}  // namespace

PBE_EXPORT int pbe_latent_prepare(const void* proj, int ld, int dtype, int q_off, int q_rank, int c_off, int rank,
                                  int r_off, int rot, const float* q_gain, const float* c_gain, const float* inv_freq,
                                  int rot_dims, float rot_scale, const int32_t* positions, const int32_t* slots,
                                  void* q_lat, void* cache, float eps, int T, cudaStream_t stream) {
  if (T <= 0) return 0;
  PrepareParams p{proj, ld, q_off, q_rank, c_off, rank, r_off, rot, q_gain, c_gain, inv_freq, rot_dims, rot_scale,
                  positions,
                  slots, q_lat, cache, eps};
  const int widest = q_rank > rank ? q_rank : rank;
  const int threads = widest >= 1024 ? 256 : 128;
  if (dtype == PBE_F32) launch_k(latent_prepare_kernel<float>, T, threads, 0, stream, p);
  else launch_k(latent_prepare_kernel<__nv_bfloat16>, T, threads, 0, stream, p);
  return launch_status();
}

// a_dtype: dtype of a; w_dtype: of the weights and of the gate; out_dtype: of the result
PBE_EXPORT int pbe_head_product(const void* a, int lda, int ha, int a_dtype, const void* w, long long hw, int wk, int wn,
                                int w_dtype, void* out, int ldo, int ho, int out_dtype, int T, int H, int K, int N,
                                int rot, int rot_dims, const float* inv_freq, const int32_t* positions,
                                const void* gate, int ldg, float rot_scale, int gate_each, cudaStream_t stream) {
  if (T <= 0 || H <= 0) return 0;
  HeadProductParams p{a, lda, ha, w, hw, wk, wn, out, ldo, ho, T, H, K, N, rot, rot_dims, inv_freq, positions, gate, ldg,
                      rot_scale, gate_each};
  dim3 grid((T + HP_TM - 1) / HP_TM, H, (N + HP_TN - 1) / HP_TN);
  if (grid.z == 0) grid.z = 1;
  const int code = a_dtype * 4 + w_dtype * 2 + out_dtype;
  switch (code) {
    case 0: launch_k(head_product_kernel<float, float, float>, grid, 256, 0, stream, p); break;
    case 4 + 2 + 0: launch_k(head_product_kernel<__nv_bfloat16, __nv_bfloat16, float>, grid, 256, 0, stream, p); break;
    case 0 + 2 + 1: launch_k(head_product_kernel<float, __nv_bfloat16, __nv_bfloat16>, grid, 256, 0, stream, p); break;
    case 4 + 2 + 1:
      launch_k(head_product_kernel<__nv_bfloat16, __nv_bfloat16, __nv_bfloat16>, grid, 256, 0, stream, p); break;
    default: return (int)cudaErrorInvalidValue;
  }
  return launch_status();
}

// tensor_cores: bfloat16 caches with rows a multiple of 16 values wide take the mma.sync kernel
// (1: blocks of 16 rows, for decoded tokens; 2: blocks of 64 rows, for prompt portions)
// sub: blocks that share a key split (tensor-core kernel only; the partial buffers then hold max_splits * sub slots)
PBE_EXPORT int pbe_latent_attention(const AttnParams* params, const float* sink, int dk, int dv, int num_work,
                                    int cache_dtype, int tensor_cores, int sub, cudaStream_t stream) {
  if (num_work <= 0) return 0;
  LatentAttnParams lp{*params, sink, dk, dv, sub < 1 ? 1 : sub};
  if (lp.a.tile_rows % LA_BM != 0 || lp.a.split_keys % LA_BN != 0 || dv > dk) return (int)cudaErrorInvalidValue;
  const bool mma = tensor_cores && cache_dtype == PBE_BF16 && dk % 16 == 0;
  if (lp.sub > 1 && (!mma || lp.a.split_keys % (lp.sub * LM_BN) != 0)) return (int)cudaErrorInvalidValue;
  if (mma) return dispatch_latent_mma(lp, num_work, tensor_cores == 2, stream);
  return cache_dtype == PBE_F32 ? dispatch_latent<float>(lp, num_work, stream)
                                : dispatch_latent<__nv_bfloat16>(lp, num_work, stream);
}

PBE_EXPORT int pbe_latent_merge(const AttnMergeParams* params, const float* sink, int sub, int split_rows,
                                cudaStream_t stream) {
  if (split_rows <= 0) return 0;
  LatentMergeParams lp{*params, sink, sub < 1 ? 1 : sub};
  dim3 grid(split_rows, lp.m.num_heads);
  const size_t smem = sizeof(float) * (size_t)lp.m.max_splits;
  if (smem > 48 * 1024) return (int)cudaErrorInvalidValue;
  const int threads = lp.m.head_dim > 256 ? 512 : (lp.m.head_dim > 128 ? 256 : (lp.m.head_dim > 64 ? 128 : 64));
  launch_k(latent_merge_kernel, grid, threads, smem, stream, lp);
  return launch_status();
}
