// Grouped-query softmax attention over the paged cache with per-head query/key norms, keys and
// values of different widths, and a choice of what a row sees and what joins its softmax:
//
//   * mask: every earlier key, the last W keys (sliding window), or the earlier keys of the
//     row's own chunk of C positions (chunks counted from position 0 of the sequence);
//   * a bias per (head, distance) added to the scaled score: bias[h][min(i - j, rows - 1)], a table
//     the host expands from whatever rule the model has (buckets, slopes ...);
//   * a unit sink: one more term e^0 in the softmax's denominator that carries no value;
//   * a gate: the output of head h, element e, times sigmoid(gate[t][h * E + e]).
//
// head_norm_write: per token, the projection's bias, an RMS norm over each head's D query or key
//   elements with one gain vector shared by the heads (float32 throughout), optionally a factor per
//   query head (a learned temperature), queries out in float32, keys and values into the pages.
// masked_attention: the float32-arithmetic kernel.  It reads the engine's attention work list
//   (request, row tile, key split, splits): the rows of a request are packed with the query heads
//   that share a key/value head, 16 packed rows a block, 32 keys a tile (a key a lane), online
//   softmax.  Scores, maxima, sums and weights are float32; queries are float32, keys and values
//   what the cache holds.
// masked_merge: the key splits of a row put together, with the sink and the gate.
#include "attention_params.cuh"
#include "common.cuh"
#include "masked_attention.cuh"
#include "pdl.cuh"

using namespace pbe;

namespace {

// ------------------------------------------------------------------ head_norm_write
struct HeadNormParams {
  const void* proj;          // [T, ld]: queries at column q_off, keys at k_off, values at v_off
  int ld, q_off, k_off, v_off;
  const float* bias;         // indexed like the projection's columns, or null
  const float* q_gain;       // [D] or null: no norm
  const float* k_gain;       // [D] or null
  const float* q_head_scale; // [H] or null: head h's normed query is multiplied by it (a temperature per head)
  const int32_t* slots;      // [T] page * page_tokens + offset; negative: nothing is written
  float* q_out;              // [T, H * D]
  void* k_pages;             // [page][G][page_tokens][D] or null
  void* v_pages;             // [page][G][page_tokens][E]
  int H, G, D, E, page_tokens;
  float eps;
};

constexpr int HN_MAX = 8;    // elements of a head a lane holds at most (D <= 256)

template <typename T>
__global__ void __launch_bounds__(128) head_norm_write_kernel(HeadNormParams p) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int H = p.H, G = p.G, D = p.D, E = p.E, PT = p.page_tokens;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const T* row = (const T*)p.proj + (size_t)t * p.ld;
  const int slot = p.slots ? p.slots[t] : -1;
  const bool store = slot >= 0 && p.k_pages != nullptr;
  const int page = store ? slot / PT : 0, off = store ? slot - page * PT : 0;
  for (int hh = warp; hh < H + G; hh += 4) {
    const bool is_q = hh < H;
    const int head = is_q ? hh : hh - H;
    if (!is_q && !store) continue;
    const int col = (is_q ? p.q_off : p.k_off) + head * D;
    const float* gain = is_q ? p.q_gain : p.k_gain;
    float x[HN_MAX];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < HN_MAX; ++i) {
      const int d = lane + i * 32;
      x[i] = 0.f;
      if (d < D) {
        x[i] = to_float(row[col + d]) + (p.bias ? p.bias[col + d] : 0.f);
        ss = fmaf(x[i], x[i], ss);
      }
    }
    float sc = 1.f;
    if (gain) sc = 1.0f / sqrtf(warp_sum(ss) / (float)D + p.eps);
#pragma unroll
    for (int i = 0; i < HN_MAX; ++i) {
      const int d = lane + i * 32;
      if (d < D) {
        float y = gain ? (x[i] * sc) * gain[d] : x[i];
        if (is_q && p.q_head_scale) y *= p.q_head_scale[head];
        if (is_q) p.q_out[((size_t)t * H + head) * D + d] = y;
        else ((T*)p.k_pages)[(((size_t)page * G + head) * PT + off) * D + d] = from_float<T>(y);
      }
    }
  }
  if (store && p.v_pages) {
    for (int i = threadIdx.x; i < G * E; i += blockDim.x) {
      const int head = i / E, e = i - head * E;
      const float y = to_float(row[p.v_off + i]) + (p.bias ? p.bias[p.v_off + i] : 0.f);
      ((T*)p.v_pages)[(((size_t)page * G + head) * PT + off) * E + e] = from_float<T>(y);
    }
  }
}

// ------------------------------------------------------------------ masked_attention
constexpr int BM = 16;       // packed rows per block
constexpr int BN = 32;       // keys per tile, one per lane
constexpr int NWARPS = 4;
constexpr int ROWS_PER_WARP = BM / NWARPS;

template <typename T, int EPL>
__global__ void __launch_bounds__(NWARPS * 32) masked_attention_kernel(AttnParams p, MaskedExtra x) {
  extern __shared__ __align__(16) float smem[];
  const int D = x.D, E = x.E;
  const int QS = (D + 3) & ~3;            // query rows start on 16-byte boundaries
  const int KS = D + 1;
  float* Qs = smem;                       // [BM][QS]
  float* Ks = Qs + BM * QS;               // [BN][D + 1]
  float* Vs = Ks + BN * KS;               // [BN][E]
  __shared__ long long base[BN];          // (page * G + kv head) * page_tokens + offset of key j, -1: none

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
  const int row_lo = pr0 / G;
  const int row_hi = (min(n_packed, pr0 + BM) - 1) / G;
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
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const float* q = (const float*)p.q;
  const T* kc = (const T*)p.k_cache;
  const T* vc = (const T*)p.v_cache;
  const int32_t* bt = p.block_table + (size_t)r * p.bt_stride;

  for (int idx = threadIdx.x; idx < BM * D; idx += blockDim.x) {
    const int i = idx / D, d = idx - i * D;
    const int pr = pr0 + i;
    float v = 0.f;
    if (pr < n_packed) {
      const int row = pr / G, hg = pr - row * G;
      v = q[((size_t)(qs + row) * H + kvh * G + hg) * D + d];
    }
    Qs[i * QS + d] = v;
  }

  float m_run[ROWS_PER_WARP], l_run[ROWS_PER_WARP], acc[ROWS_PER_WARP][EPL];
#pragma unroll
  for (int j = 0; j < ROWS_PER_WARP; ++j) {
    m_run[j] = -INFINITY;
    l_run[j] = 0.f;
#pragma unroll
    for (int i = 0; i < EPL; ++i) acc[j][i] = 0.f;
  }
  // this warp's rows: position and head (fixed for the block)
  int row_pos[ROWS_PER_WARP], row_head[ROWS_PER_WARP];
#pragma unroll
  for (int j = 0; j < ROWS_PER_WARP; ++j) {
    const int pr = pr0 + warp + j * NWARPS;
    row_pos[j] = pr < n_packed ? pos0 + pr / G : -1;
    row_head[j] = kvh * G + (pr < n_packed ? pr % G : 0);
  }

  const int tile0 = (k_begin / BN) * BN;
  for (int ts = tile0; ts < k_end; ts += BN) {
    __syncthreads();   // the tile before is consumed (and Qs written, first time)
    if (threadIdx.x < BN) {
      const int key = ts + threadIdx.x;
      long long b = -1;
      if (key >= k_begin && key < k_end) {
        const int page = bt[key / P];
        if (page >= 0) b = ((long long)page * KV + kvh) * P + key % P;
      }
      base[threadIdx.x] = b;
    }
    __syncthreads();
    // keys and values of the tile as float32: four elements a thread and turn where the widths allow
    if ((D & 3) == 0) {
      const int dq = D >> 2;
      for (int i = threadIdx.x; i < BN * dq; i += blockDim.x) {
        const int j = i / dq, d = (i - j * dq) * 4;
        const long long b = base[j];
        float f[4] = {0.f, 0.f, 0.f, 0.f};
        if (b >= 0) {
#pragma unroll
          for (int u = 0; u < 4; ++u) f[u] = to_float(kc[b * D + d + u]);
        }
        float* kd = Ks + j * KS + d;
        kd[0] = f[0]; kd[1] = f[1]; kd[2] = f[2]; kd[3] = f[3];
      }
    } else {
      for (int i = threadIdx.x; i < BN * D; i += blockDim.x) {
        const int j = i / D, d = i - j * D;
        const long long b = base[j];
        Ks[j * KS + d] = b >= 0 ? to_float(kc[b * D + d]) : 0.f;
      }
    }
    for (int i = threadIdx.x; i < BN * E; i += blockDim.x) {
      const int j = i / E, e = i - j * E;
      const long long b = base[j];
      Vs[i] = b >= 0 ? to_float(vc[b * E + e]) : 0.f;
    }
    __syncthreads();
    float s[ROWS_PER_WARP];
#pragma unroll
    for (int j = 0; j < ROWS_PER_WARP; ++j) s[j] = 0.f;
    {
      const float* krow = Ks + lane * KS;
      int d = 0;
      for (; d + 3 < D; d += 4) {
        const float k0 = krow[d], k1 = krow[d + 1], k2 = krow[d + 2], k3 = krow[d + 3];
#pragma unroll
        for (int j = 0; j < ROWS_PER_WARP; ++j) {
          const float4 qv = *reinterpret_cast<const float4*>(Qs + (warp + j * NWARPS) * QS + d);
          float a = s[j];
          a = fmaf(qv.x, k0, a);
          a = fmaf(qv.y, k1, a);
          a = fmaf(qv.z, k2, a);
          a = fmaf(qv.w, k3, a);
          s[j] = a;
        }
      }
      for (; d < D; ++d) {
        const float k0 = krow[d];
#pragma unroll
        for (int j = 0; j < ROWS_PER_WARP; ++j) s[j] = fmaf(Qs[(warp + j * NWARPS) * QS + d], k0, s[j]);
      }
    }
    float pj[ROWS_PER_WARP];
    const int key = ts + lane;
    const bool have = base[lane] >= 0;
#pragma unroll
    for (int j = 0; j < ROWS_PER_WARP; ++j) {
      pj[j] = 0.f;
      const int pos = row_pos[j];
      if (pos < 0) continue;
      const bool visible = have && key <= pos && key >= first_visible(pos, x.mask_kind, p.window);
      float sc = -INFINITY;
      if (visible) {
        sc = s[j] * p.scale;
        if (x.bias) sc += __ldg(x.bias + (size_t)row_head[j] * x.bias_rows + min(pos - key, x.bias_rows - 1));
      }
      const float m_new = fmaxf(m_run[j], warp_max(sc));
      if (m_new == -INFINITY) continue;     // nothing visible so far
      pj[j] = visible ? expf(sc - m_new) : 0.f;
      const float alpha = expf(m_run[j] - m_new);
      l_run[j] = l_run[j] * alpha + warp_sum(pj[j]);
      m_run[j] = m_new;
#pragma unroll
      for (int ii = 0; ii < EPL; ++ii) acc[j][ii] *= alpha;
    }
    for (int kk = 0; kk < BN; ++kk) {
      float vv[EPL];
#pragma unroll
      for (int ii = 0; ii < EPL; ++ii) {
        const int e = lane + ii * 32;
        vv[ii] = e < E ? Vs[kk * E + e] : 0.f;
      }
#pragma unroll
      for (int j = 0; j < ROWS_PER_WARP; ++j) {
        const float pk = __shfl_sync(0xffffffffu, pj[j], kk);
#pragma unroll
        for (int ii = 0; ii < EPL; ++ii) acc[j][ii] = fmaf(pk, vv[ii], acc[j][ii]);
      }
    }
  }

#pragma unroll
  for (int j = 0; j < ROWS_PER_WARP; ++j) {
    const int pr = pr0 + warp + j * NWARPS;
    if (pr >= n_packed) continue;
    const int row = pr / G;
    const int head = row_head[j];
    const int t = qs + row;
    if (nsplit <= 1) {
      float m = m_run[j], l = l_run[j], rescale = 1.f;
      if (x.unit_sink) add_unit_sink(m, l, rescale);
      const float inv = l > 0.f ? rescale / l : 0.f;
      T* o = (T*)p.out + ((size_t)t * H + head) * E;
      const T* g = x.gate ? (const T*)x.gate + (size_t)t * x.ldg + head * E : nullptr;
#pragma unroll
      for (int ii = 0; ii < EPL; ++ii) {
        const int e = lane + ii * 32;
        if (e < E) {
          float y = acc[j][ii] * inv;
          if (g) y *= sigmoidf_(to_float(g[e]));
          o[e] = from_float<T>(y);
        }
      }
    } else {
      const int srow = p.tok_split_row[t];
      const size_t b = ((size_t)srow * H + head) * p.max_splits + split;
      float* po = p.part_o + b * E;
#pragma unroll
      for (int ii = 0; ii < EPL; ++ii) {
        const int e = lane + ii * 32;
        if (e < E) po[e] = acc[j][ii];
      }
      if (lane == 0) {
        p.part_ml[b * 2] = m_run[j];
        p.part_ml[b * 2 + 1] = l_run[j];
      }
    }
  }
}

struct MaskedMergeExtra {
  int unit_sink;
  const void* gate;
  int ldg;
};

template <typename T>
__global__ void masked_merge_kernel(AttnMergeParams p, MaskedMergeExtra x) {
  pdl_launch_dependents();
  pdl_wait();
  const int srow = blockIdx.x, head = blockIdx.y;
  const int n = p.split_counts[srow];
  if (n <= 1) return;
  const int t = p.split_tokens[srow];
  const int E = p.head_dim;
  const size_t base = ((size_t)srow * p.num_heads + head) * p.max_splits;
  float m = -INFINITY;
  for (int s = 0; s < n; ++s) m = fmaxf(m, p.part_ml[(base + s) * 2]);
  if (x.unit_sink) m = fmaxf(m, 0.f);
  float l = x.unit_sink ? expf(-m) : 0.f;
  for (int s = 0; s < n; ++s) {
    const float ms = p.part_ml[(base + s) * 2];
    if (ms != -INFINITY) l += p.part_ml[(base + s) * 2 + 1] * expf(ms - m);
  }
  const float inv = l > 0.f ? 1.0f / l : 0.f;
  T* o = (T*)p.out + ((size_t)t * p.num_heads + head) * E;
  const T* g = x.gate ? (const T*)x.gate + (size_t)t * x.ldg + head * E : nullptr;
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    float a = 0.f;
    for (int s = 0; s < n; ++s) {
      const float ms = p.part_ml[(base + s) * 2];
      if (ms != -INFINITY) a += p.part_o[(base + s) * E + e] * expf(ms - m);
    }
    float y = a * inv;
    if (g) y *= sigmoidf_(to_float(g[e]));
    o[e] = from_float<T>(y);
  }
}

size_t ma_smem(int D, int E) {
  return sizeof(float) * ((size_t)BM * ((D + 3) & ~3) + (size_t)BN * (D + 1) + (size_t)BN * E);
}

template <typename T, int EPL>
int launch_ma(const AttnParams& p, const MaskedExtra& x, int num_work, cudaStream_t stream) {
  const size_t smem = ma_smem(x.D, x.E);
  static size_t opted = 48 * 1024;
  if (smem > opted) {
    cudaFuncSetAttribute(masked_attention_kernel<T, EPL>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    opted = 200 * 1024;
  }
  launch_k(masked_attention_kernel<T, EPL>, dim3(num_work, p.num_kv_heads), NWARPS * 32, smem, stream, p, x);
  return launch_status();
}

template <typename T>
int dispatch_ma(const AttnParams& p, const MaskedExtra& x, int num_work, cudaStream_t stream) {
  const int epl = (x.E + 31) / 32;
  if (epl <= 1) return launch_ma<T, 1>(p, x, num_work, stream);
  if (epl <= 2) return launch_ma<T, 2>(p, x, num_work, stream);
  if (epl <= 4) return launch_ma<T, 4>(p, x, num_work, stream);
  return launch_ma<T, 8>(p, x, num_work, stream);
}
}  // namespace

PBE_EXPORT int pbe_masked_attention_tile_rows() { return BM; }
PBE_EXPORT int pbe_masked_attention_key_tile() { return BN; }

PBE_EXPORT int pbe_head_norm_write(const void* proj, int ld, int q_off, int k_off, int v_off, const float* bias,
                                   const float* q_gain, const float* k_gain, const float* q_head_scale,
                                   const int32_t* slots, float* q_out,
                                   void* k_pages, void* v_pages, int T, int H, int G, int D, int E, int page_tokens,
                                   float eps, int dtype, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (D > 32 * HN_MAX || D < 1 || E < 1) return (int)cudaErrorInvalidValue;
  HeadNormParams p{proj, ld, q_off, k_off, v_off, bias, q_gain, k_gain, q_head_scale, slots, q_out, k_pages, v_pages,
                   H, G, D, E, page_tokens, eps};
  if (dtype == PBE_F32) launch_k(head_norm_write_kernel<float>, T, 128, 0, stream, p);
  else launch_k(head_norm_write_kernel<__nv_bfloat16>, T, 128, 0, stream, p);
  return launch_status();
}

PBE_EXPORT int pbe_masked_attention(const AttnParams* params, int D, int E, const float* bias, int bias_rows,
                                    int mask_kind, int unit_sink, const void* gate, int ldg, int num_work,
                                    int dtype, cudaStream_t stream) {
  if (num_work <= 0) return 0;
  AttnParams p = *params;
  if (p.num_heads % p.num_kv_heads != 0 || p.tile_rows != BM || p.split_keys % BN != 0 || D < 1 || E < 1 ||
      E > 256 || mask_kind < 0 || mask_kind > 2 || (mask_kind != 0 && p.window < 1) || (bias && bias_rows < 1))
    return (int)cudaErrorInvalidValue;
  if (ma_smem(D, E) > 200 * 1024) return (int)cudaErrorInvalidValue;
  MaskedExtra x{bias, bias_rows, mask_kind, unit_sink, gate, ldg, D, E};
  return dtype == PBE_F32 ? dispatch_ma<float>(p, x, num_work, stream)
                          : dispatch_ma<__nv_bfloat16>(p, x, num_work, stream);
}

PBE_EXPORT int pbe_masked_merge(const AttnMergeParams* params, int unit_sink, const void* gate, int ldg,
                                int split_rows, int dtype, cudaStream_t stream) {
  if (split_rows <= 0) return 0;
  AttnMergeParams p = *params;
  MaskedMergeExtra x{unit_sink, gate, ldg};
  dim3 grid(split_rows, p.num_heads);
  const int threads = p.head_dim > 64 ? 128 : 64;
  if (dtype == PBE_F32) launch_k(masked_merge_kernel<float>, grid, threads, 0, stream, p, x);
  else launch_k(masked_merge_kernel<__nv_bfloat16>, grid, threads, 0, stream, p, x);
  return launch_status();
}
