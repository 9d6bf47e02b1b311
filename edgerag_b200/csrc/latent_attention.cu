// Attention through a latent: per token the cache holds ONE row [c (R) | kr (dr)], the normed
// low-rank latent that every head's keys and values are made from and one rotated key part that all
// heads share.  The heads' up-projections are folded into the queries and the outputs
// ("absorbed"): with  qa_h = W_uk_h^T q_h^unrotated  (R wide)
//     score(h, j) = (qa_h . c_j + q_h^rotated . kr_j) * scale,     o_h = W_uv_h (sum_j p_hj c_j),
// so the kernel is multi-query attention whose key row is the cache row (Dk = R + dr) and whose
// value row is the first R entries of the same row: a key is read once and serves both products and
// every head.  Nothing is up-projected per cached token.
//
// Kernels (all float arithmetic; T is the cache's and the projections' element type):
//   latent_store_kernel      unit-RMS norm of the down-projection's first R entries times a plain weight,
//                            pairwise rotation of its last dr entries, both written to the token's cache
//                            row; optionally the same norm for a query latent.
//   latent_q_rotate_kernel   the rotated part of every head's query, written as float beside the
//                            absorbed part.
//   latent_attention_kernel  one warp per (token, head): online softmax over the visible keys (or over
//                            one split of them), an optional sink in the denominator, an optional
//                            sigmoid gate per head on the result.
//   latent_combine_kernel    merges the splits of a row in split order.
// Rotation convention: neighbouring pairs (2i, 2i+1), angle = position * inv_freq[i] in float.
#include "common.cuh"

using namespace erb;

ERB_DEFINE_LAST_ERROR(erb_last_error)

namespace {

template <typename T> struct Pair;   // two neighbouring elements as floats
template <> struct Pair<float> {
  static __device__ __forceinline__ float2 load(const float* p) { return *reinterpret_cast<const float2*>(p); }
};
template <> struct Pair<__nv_bfloat16> {
  static __device__ __forceinline__ float2 load(const __nv_bfloat16* p) {
    return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p));
  }
};

// ---------------------------------------------------------------------------------------------
// One block per token.  `proj` is the token's row of the fused input projection.
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(128)
latent_store_kernel(const T* __restrict__ proj, int ld, int off_kv, int R, int dr, const float* __restrict__ kv_weight,
                    float eps, const int* __restrict__ positions, const float* __restrict__ inv_freq, int rot_dims,
                    const int* __restrict__ slots, T* __restrict__ pages, int off_q, int q_rank,
                    const float* __restrict__ q_weight, T* __restrict__ q_latent) {
  chain_wait();
  __shared__ float scratch[32];
  const int t = blockIdx.x;
  const T* row = proj + (size_t)t * ld;
  if (off_kv >= 0) {
    const T* x = row + off_kv;
    float ss = 0.f;
    for (int i = threadIdx.x; i < R; i += blockDim.x) {
      const float v = Elem<T>::load(x + i);
      ss += v * v;
    }
    const float rs = rsqrtf(block_sum(ss, scratch) / (float)R + eps);
    const int slot = slots[t];
    if (slot >= 0) {
      T* dst = pages + (size_t)slot * (R + dr);
      for (int i = threadIdx.x; i < R; i += blockDim.x) Elem<T>::store(dst + i, Elem<T>::load(x + i) * rs * kv_weight[i]);
      const float pos = (float)positions[t];
      for (int i = threadIdx.x; i < dr / 2; i += blockDim.x) {
        float u = Elem<T>::load(x + R + 2 * i), v = Elem<T>::load(x + R + 2 * i + 1);
        if (2 * i < rot_dims) {
          float sn, cs;
          sincosf(pos * inv_freq[i], &sn, &cs);
          const float a = u * cs - v * sn, b = v * cs + u * sn;
          u = a; v = b;
        }
        Elem<T>::store(dst + R + 2 * i, u);
        Elem<T>::store(dst + R + 2 * i + 1, v);
      }
    }
  }
  if (q_rank > 0) {
    const T* x = row + off_q;
    float ss = 0.f;
    for (int i = threadIdx.x; i < q_rank; i += blockDim.x) {
      const float v = Elem<T>::load(x + i);
      ss += v * v;
    }
    const float rs = rsqrtf(block_sum(ss, scratch) / (float)q_rank + eps);
    T* dst = q_latent + (size_t)t * q_rank;
    for (int i = threadIdx.x; i < q_rank; i += blockDim.x) Elem<T>::store(dst + i, Elem<T>::load(x + i) * rs * q_weight[i]);
  }
}

// q rows [tokens][ld] hold, per head, dn unrotated then dr rotated entries; the rotated ones go, turned,
// to q_lat[token][head][R .. R + dr) as float.
template <typename T>
__global__ void __launch_bounds__(128)
latent_q_rotate_kernel(const T* __restrict__ q, int ld, int H, int dn, int dr, int R, const int* __restrict__ positions,
                       const float* __restrict__ inv_freq, int rot_dims, float* __restrict__ q_lat) {
  chain_wait();
  const int t = blockIdx.x;
  const float pos = (float)positions[t];
  const int half = dr / 2;
  for (int idx = threadIdx.x; idx < H * half; idx += blockDim.x) {
    const int h = idx / half, i = idx % half;
    const T* src = q + (size_t)t * ld + (size_t)h * (dn + dr) + dn + 2 * i;
    float u = Elem<T>::load(src), v = Elem<T>::load(src + 1);
    if (2 * i < rot_dims) {
      float sn, cs;
      sincosf(pos * inv_freq[i], &sn, &cs);
      const float a = u * cs - v * sn, b = v * cs + u * sn;
      u = a; v = b;
    }
    float* dst = q_lat + ((size_t)t * H + h) * (R + dr) + R + 2 * i;
    dst[0] = u;
    dst[1] = v;
  }
}

constexpr int kLatWarps = 4;    // (token, head) rows per block: neighbouring heads of a token share its keys in L1
constexpr int kLatKeys = 4;     // keys in flight per warp

// The softmax state of one row after its keys (or one split of them): running maximum, denominator,
// unnormalised sum of latents.  Finishing folds in the sink (a term exp(sink) of the denominator with
// no key and no value) and the head's gate.
__device__ __forceinline__ float finish_factor(float m, float l, const float* sink, int h, float gate_logit, bool gated) {
  float f;
  if (sink) {
    const float s = sink[h], top = fmaxf(m, s);
    const float e = (m == -INFINITY) ? 0.f : expf(m - top);
    f = e / (l * e + expf(s - top));
  } else {
    f = 1.f / l;
  }
  if (gated) f *= 1.f / (1.f + expf(-gate_logit));
  return f;
}

// NI: pairs of the cache row per lane (Dk <= 64 * NI).
template <typename T, int NI>
__global__ void __launch_bounds__(kLatWarps * 32)
latent_attention_kernel(const float* __restrict__ q_lat, const T* __restrict__ pages, const int* __restrict__ block_tables,
                        int max_pages, const int* __restrict__ seq_of_token, const int* __restrict__ positions,
                        const T* __restrict__ gate, int gate_ld, const float* __restrict__ sink, T* __restrict__ out,
                        float* __restrict__ part, int first_token, int n_rows, int H, int R, int Dk, int page_size,
                        int split_keys, int n_splits, float scale, int window) {
  chain_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row = blockIdx.x * kLatWarps + warp;
  if (row >= n_rows) return;                       // warps are independent: no block-wide barrier below
  const int split = blockIdx.y;
  const int t = first_token + row / H, h = row % H;
  const int seq = seq_of_token[t], pos = positions[t];
  // a window moves the first key; the splits stay at multiples of their size, counted from the one that holds it
  const int lo = first_visible_key(pos, window);
  const int base = n_splits > 1 ? (lo / split_keys + split) * split_keys : 0;
  const int begin = n_splits > 1 ? max(lo, base) : lo;
  const int end = n_splits > 1 ? min(pos + 1, base + split_keys) : pos + 1;

  float2 q[NI], acc[NI];
  const float* q_row = q_lat + ((size_t)t * H + h) * Dk;
#pragma unroll
  for (int i = 0; i < NI; ++i) {
    const int e = 2 * (lane + 32 * i);
    q[i] = e < Dk ? *reinterpret_cast<const float2*>(q_row + e) : make_float2(0.f, 0.f);
    q[i].x *= scale; q[i].y *= scale;
    acc[i] = make_float2(0.f, 0.f);
  }
  float m = -INFINITY, l = 0.f;
  const int* bt = block_tables + (size_t)seq * max_pages;
  for (int k0 = begin; k0 < end; k0 += kLatKeys) {
    float2 kv[kLatKeys][NI];
    float s[kLatKeys];
#pragma unroll
    for (int j = 0; j < kLatKeys; ++j) {
      const int k = k0 + j < end ? k0 + j : k0;   // (a key past the end is read as the first of the group and masked)
      const T* key = pages + ((size_t)bt[k / page_size] * page_size + k % page_size) * Dk;
      float sum = 0.f;
#pragma unroll
      for (int i = 0; i < NI; ++i) {
        const int e = 2 * (lane + 32 * i);
        kv[j][i] = e < Dk ? Pair<T>::load(key + e) : make_float2(0.f, 0.f);
        sum = fmaf(q[i].x, kv[j][i].x, sum);
        sum = fmaf(q[i].y, kv[j][i].y, sum);
      }
      s[j] = sum;
    }
    float top = m;
#pragma unroll
    for (int j = 0; j < kLatKeys; ++j) {
      s[j] = warp_sum(s[j]);
      if (k0 + j >= end) s[j] = -INFINITY;
      top = fmaxf(top, s[j]);
    }
    const float alpha = (m == -INFINITY) ? 0.f : expf(m - top);
    float p[kLatKeys], psum = 0.f;
#pragma unroll
    for (int j = 0; j < kLatKeys; ++j) {
      p[j] = expf(s[j] - top);                    // exp(-inf) = 0 for masked keys
      psum += p[j];
    }
    l = l * alpha + psum;
#pragma unroll
    for (int i = 0; i < NI; ++i) {
      float ax = acc[i].x * alpha, ay = acc[i].y * alpha;
#pragma unroll
      for (int j = 0; j < kLatKeys; ++j) {
        ax = fmaf(p[j], kv[j][i].x, ax);
        ay = fmaf(p[j], kv[j][i].y, ay);
      }
      acc[i] = make_float2(ax, ay);
    }
    m = top;
  }
  if (n_splits > 1) {
    float* dst = part + ((size_t)row * n_splits + split) * (R + 2);
    if (lane == 0) { dst[0] = m; dst[1] = l; }
#pragma unroll
    for (int i = 0; i < NI; ++i) {
      const int e = 2 * (lane + 32 * i);
      if (e < R) { dst[2 + e] = acc[i].x; dst[3 + e] = acc[i].y; }
    }
    return;
  }
  const float f = finish_factor(m, l, sink, h, gate ? Elem<T>::load(gate + (size_t)t * gate_ld + h) : 0.f, gate != nullptr);
  T* o = out + ((size_t)t * H + h) * R;
#pragma unroll
  for (int i = 0; i < NI; ++i) {
    const int e = 2 * (lane + 32 * i);
    if (e < R) { Elem<T>::store(o + e, acc[i].x * f); Elem<T>::store(o + e + 1, acc[i].y * f); }
  }
}

// The splits' states of a row merged in split order (a split the row does not reach has l = 0).
// The splits' maxima and denominators are fetched by one thread each; every split's weight exp(m_s - m) is
// taken once and shared.  At most kCombineSplits splits.
constexpr int kCombineSplits = 128;
template <typename T>
__global__ void __launch_bounds__(128)
latent_combine_kernel(const float* __restrict__ part, const T* __restrict__ gate, int gate_ld, const float* __restrict__ sink,
                      T* __restrict__ out, int first_token, int H, int R, int n_splits) {
  chain_wait();
  __shared__ float m_s[kCombineSplits], l_s[kCombineSplits], weight[kCombineSplits];
  const int row = blockIdx.x;
  const int t = first_token + row / H, h = row % H;
  const size_t stride = (size_t)(R + 2);
  const float* src = part + (size_t)row * n_splits * stride;
  float l_mine = 0.f;
  if ((int)threadIdx.x < n_splits) {
    m_s[threadIdx.x] = src[threadIdx.x * stride];
    l_mine = src[threadIdx.x * stride + 1];
  }
  __syncthreads();
  float m = -INFINITY;
  for (int s = 0; s < n_splits; ++s) m = fmaxf(m, m_s[s]);
  if ((int)threadIdx.x < n_splits) {
    const float w = m_s[threadIdx.x] == -INFINITY ? 0.f : expf(m_s[threadIdx.x] - m);
    weight[threadIdx.x] = w;
    l_s[threadIdx.x] = l_mine * w;
  }
  __syncthreads();
  float l = 0.f;
  for (int s = 0; s < n_splits; ++s) l += l_s[s];
  const float f = finish_factor(m, l, sink, h, gate ? Elem<T>::load(gate + (size_t)t * gate_ld + h) : 0.f, gate != nullptr);
  T* o = out + ((size_t)t * H + h) * R;
  // (gridDim.y blocks share a row, 128 neighbouring columns at a time each: a thread then has one column and its
  // loads of all splits in flight, instead of a walk over several columns one after the other)
  for (int e = blockIdx.y * blockDim.x + threadIdx.x; e < R; e += gridDim.y * blockDim.x) {
    float sum = 0.f;
#pragma unroll 8
    for (int s = 0; s < n_splits; ++s) sum = fmaf(src[s * stride + 2 + e], weight[s], sum);
    Elem<T>::store(o + e, sum * f);
  }
}

#if ERB_ELEM == 1
// ---------------------------------------------------------------------------------------------
// The same attention on tensor cores (bfloat16): a block owns M = 16 * MT neighbouring (token, head) rows of
// one sequence and walks the sequence's cache rows in tiles of 64 keys, which arrive by 16-byte
// asynchronous copies straight from the pages into one of two stages of shared memory (keys past the
// end are filled with zeros).  Per tile: warp w makes the scores of the tile's keys 8w .. 8w + 7 for all M
// rows (mma.sync m16n8k16, queries and keys by ldmatrix, float accumulation over the whole cache row; with two
// row tiles the block has sixteen warps and a pair of warps shares a group of keys, one row tile each);
// the groups' maxima and sums of a row go through shared memory to the one thread that keeps the row's
// running maximum and denominator and hands back the new maximum and the rescaling factor; the weights go
// to shared memory as bfloat16; then
// every warp adds  P [M x 64] . C [64 x its NT * 8 columns of the latent]  to its float accumulators, the
// latent read from the same stage by ldmatrix.trans.  Queries are scaled, rounded to bfloat16 and kept in
// shared memory for the whole walk.  Splits, sink and gate are those of the kernel above.
// ---------------------------------------------------------------------------------------------
constexpr int kMmaKeyGroups = 8;   // groups of 8 keys in a tile: one per warp, or per pair of warps
constexpr int kMmaKeys = 64;
constexpr int kMmaPStride = kMmaKeys + 8;

__device__ __forceinline__ void ldsm4(uint32_t* r, const void* p) {
  const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void ldsm4t(uint32_t* r, const void* p) {
  const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void ldsm4s(uint32_t* r, uint32_t a) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void mma16816(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void copy16(void* dst, const void* src, bool real) {
  const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
  const int bytes = real ? 16 : 0;                           // 0 bytes read: the 16 bytes are filled with zeros
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(bytes) : "memory");
}

template <int MT, int NT, int W>
__global__ void __launch_bounds__(W * 32, 1)
latent_attention_mma_kernel(const float* __restrict__ q_lat, const __nv_bfloat16* __restrict__ pages,
                            const int* __restrict__ block_tables, int max_pages, const int* __restrict__ seq_starts,
                            const int* __restrict__ positions, const __nv_bfloat16* __restrict__ gate, int gate_ld,
                            const float* __restrict__ sink, __nv_bfloat16* __restrict__ out, float* __restrict__ part,
                            int first_token, int seq0, int n_seqs, int H, int R, int Dk, int page_size, int split_keys,
                            int n_splits, float scale, int window) {
  chain_wait();
  constexpr int M = 16 * MT;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int D16 = (Dk + 15) & ~15, DkP = D16 + 8;
  __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(smem_raw);        // [M][DkP]
  __nv_bfloat16* Ks = Qs + M * DkP;                                      // [2][64][DkP]
  __nv_bfloat16* Ps = Ks + 2 * kMmaKeys * DkP;                           // [M][72]
  float* red_max = reinterpret_cast<float*>(Ps + M * kMmaPStride);       // [key groups][M]
  float* red_sum = red_max + kMmaKeyGroups * M;                          // [key groups][M]
  float* row_top = red_sum + kMmaKeyGroups * M;                          // [M]: a row's maximum so far (at the end: its final one)
  float* row_alpha = row_top + M;                                        // [M]: what the tile rescales the row by (at the end: its sum)
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, tq = lane & 3;

  // which sequence, which of its row tiles
  int tile = blockIdx.x, s = seq0, rows_s = 0;
  for (;; ++s) {
    if (s >= seq0 + n_seqs) return;
    rows_s = (seq_starts[s + 1] - seq_starts[s]) * H;
    const int tiles = (rows_s + M - 1) / M;
    if (tile < tiles) break;
    tile -= tiles;
  }
  const int tok0 = seq_starts[s], r0 = tile * M;
  const int valid = min(M, rows_s - r0);
  const int pos_max = positions[tok0 + (r0 + valid - 1) / H];
  const int split = blockIdx.y;
  // the first key any row of the block sees (its first row's window); splits are counted from the one that holds it
  const int lo = first_visible_key(positions[tok0 + r0 / H], window);
  const int base = n_splits > 1 ? (lo / split_keys + split) * split_keys : 0;
  const int begin = n_splits > 1 ? max(lo, base) : lo;
  const int end = n_splits > 1 ? min(pos_max + 1, base + split_keys) : pos_max + 1;
  const int* bt = block_tables + (size_t)s * max_pages;
  const int page_shift = (page_size & (page_size - 1)) == 0 ? __ffs(page_size) - 1 : -1;

  // queries: scaled, rounded, zero beyond the valid rows and beyond Dk
  const float* q_rows = q_lat + ((size_t)tok0 * H + r0) * Dk;
  for (int idx = threadIdx.x; idx < M * (D16 / 2); idx += blockDim.x) {
    const int r = idx / (D16 / 2), c = 2 * (idx % (D16 / 2));
    float2 v = make_float2(0.f, 0.f);
    if (r < valid && c < Dk) v = *reinterpret_cast<const float2*>(q_rows + (size_t)r * Dk + c);
    *reinterpret_cast<__nv_bfloat162*>(Qs + r * DkP + c) = __floats2bfloat162_rn(v.x * scale, v.y * scale);
  }
  if (D16 > Dk) {          // the copies never touch these columns
    for (int idx = threadIdx.x; idx < 2 * kMmaKeys * (D16 - Dk); idx += blockDim.x)
      Ks[(idx / (D16 - Dk)) * DkP + Dk + idx % (D16 - Dk)] = __float2bfloat16_rn(0.f);
  }

  int pos_r[MT][2];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const int r = 16 * mt + g + 8 * j;
      pos_r[mt][j] = r < valid ? positions[tok0 + (r0 + r) / H] : -1;
    }
  // Row r's running maximum and denominator are kept by thread r alone (the first M threads of the block), which
  // also tells the others, per tile, the new maximum and the factor that rescales what has been summed so far.
  float m_own = -INFINITY, l_own = 0.f, alpha_own = 1.f;
  float o[MT][NT][4];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int i = 0; i < 4; ++i) o[mt][nt][i] = 0.f;

  // A tile's rows are shared out by warp (rows warp, warp + 8, ...), a row's 16-byte pieces by lane: one page
  // lookup per row and no division per piece.
  const int chunks_per_row = Dk / 8;
  auto load_tile = [&](int k0, int stage) {
    __nv_bfloat16* dst = Ks + stage * kMmaKeys * DkP;
#pragma unroll 2
    for (int r = warp; r < kMmaKeys; r += W) {
      const int k = k0 + r;
      const bool real = k < end;
      const __nv_bfloat16* src = pages;
      if (real) {
        const int page = page_shift >= 0 ? k >> page_shift : k / page_size;       // (pages of a power of two: no division)
        src = pages + ((size_t)bt[page] * page_size + (k - page * page_size)) * Dk;
      }
      __nv_bfloat16* drow = dst + r * DkP;
      for (int c = lane; c < chunks_per_row; c += 32) copy16(drow + 8 * c, real ? src + 8 * c : src, real);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };

  const int n_tiles = begin < end ? (end - begin + kMmaKeys - 1) / kMmaKeys : 0;
  if (n_tiles > 0) load_tile(begin, 0);
  for (int it = 0; it < n_tiles; ++it) {
    const int k0 = begin + it * kMmaKeys, stage = it & 1;
    if (it + 1 < n_tiles) {
      load_tile(k0 + kMmaKeys, stage ^ 1);
      asm volatile("cp.async.wait_group 1;" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    __syncthreads();
    const __nv_bfloat16* Kt = Ks + stage * kMmaKeys * DkP;

    // Scores of one group of 8 keys.  With 8 warps a warp takes its group for all row tiles; with 16 (two row
    // tiles) warps 2 kg and 2 kg + 1 take group kg for one row tile each.  The sum over the row's entries runs in
    // four chains (k-steps 0, 1, 2, 3 mod 4), so that a product does not wait for the one before it.
    constexpr int QM = W == 16 ? 1 : MT;                      // row tiles a warp makes scores for
    const int mt0 = W == 16 ? (warp & 1) : 0, kg = W == 16 ? (warp >> 1) : warp;
    float ch[QM][4][4];
#pragma unroll
    for (int q = 0; q < QM; ++q)
#pragma unroll
      for (int c = 0; c < 4; ++c)
#pragma unroll
        for (int i = 0; i < 4; ++i) ch[q][c][i] = 0.f;
    const uint32_t kb = (uint32_t)__cvta_generic_to_shared(Kt + (8 * kg + (lane & 7)) * DkP + 8 * (lane >> 3));
    const uint32_t qb = (uint32_t)__cvta_generic_to_shared(Qs + (16 * mt0 + (lane & 7) + 8 * ((lane >> 3) & 1)) * DkP + 8 * (lane >> 4));
    const uint32_t q_tile = 16 * DkP * (uint32_t)sizeof(__nv_bfloat16);
#pragma unroll 2
    for (int kk = 0; kk < D16; kk += 64) {
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const int k32 = kk + 32 * half;
        if (k32 < D16) {
          uint32_t b[4];
          ldsm4s(b, kb + 2 * k32);
          const bool second = k32 + 16 < D16;
#pragma unroll
          for (int q = 0; q < QM; ++q) {
            uint32_t a[4];
            ldsm4s(a, qb + q * q_tile + 2 * k32);
            mma16816(ch[q][2 * half], a, b[0], b[1]);
            if (second) {
              ldsm4s(a, qb + q * q_tile + 2 * k32 + 32);
              mma16816(ch[q][2 * half + 1], a, b[2], b[3]);
            }
          }
        }
      }
    }
    float sc[QM][4];
#pragma unroll
    for (int q = 0; q < QM; ++q)
#pragma unroll
      for (int i = 0; i < 4; ++i) sc[q][i] = (ch[q][0][i] + ch[q][1][i]) + (ch[q][2][i] + ch[q][3][i]);
    const int key0 = k0 + 8 * kg + 2 * tq;
#pragma unroll
    for (int q = 0; q < QM; ++q)
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const int pos_row = W == 16 ? (mt0 ? pos_r[MT - 1][j] : pos_r[0][j]) : pos_r[q][j];
        const int lim = min(pos_row, end - 1), low = first_visible_key(pos_row, window);
        if (key0 > lim || key0 < low) sc[q][2 * j] = -INFINITY;
        if (key0 + 1 > lim || key0 + 1 < low) sc[q][2 * j + 1] = -INFINITY;
        float mx = fmaxf(sc[q][2 * j], sc[q][2 * j + 1]);
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        if (tq == 0) red_max[kg * M + 16 * (mt0 + q) + g + 8 * j] = mx;
      }
    __syncthreads();
    if ((int)threadIdx.x < M) {
      const int r = threadIdx.x;
      float top = m_own;
#pragma unroll
      for (int w = 0; w < kMmaKeyGroups; ++w) top = fmaxf(top, red_max[w * M + r]);
      alpha_own = (top == -INFINITY) ? 1.f : (m_own == -INFINITY ? 0.f : __expf(m_own - top));
      m_own = top;
      row_top[r] = top;
      row_alpha[r] = alpha_own;
    }
    __syncthreads();
#pragma unroll
    for (int q = 0; q < QM; ++q)
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const int r = 16 * (mt0 + q) + g + 8 * j;
        const float top = row_top[r];
        const bool none = top == -INFINITY;
        const float p0 = (none || sc[q][2 * j] == -INFINITY) ? 0.f : __expf(sc[q][2 * j] - top);
        const float p1 = (none || sc[q][2 * j + 1] == -INFINITY) ? 0.f : __expf(sc[q][2 * j + 1] - top);
        *reinterpret_cast<__nv_bfloat162*>(Ps + r * kMmaPStride + 8 * kg + 2 * tq) = __floats2bfloat162_rn(p0, p1);
        float ps = p0 + p1;
        ps += __shfl_xor_sync(0xffffffffu, ps, 1);
        ps += __shfl_xor_sync(0xffffffffu, ps, 2);
        if (tq == 0) red_sum[kg * M + r] = ps;
      }
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const float alpha = row_alpha[16 * mt + g + 8 * j];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          o[mt][nt][2 * j] *= alpha;
          o[mt][nt][2 * j + 1] *= alpha;
        }
      }
    __syncthreads();
    if ((int)threadIdx.x < M) {
      float sum = 0.f;
#pragma unroll
      for (int w = 0; w < kMmaKeyGroups; ++w) sum += red_sum[w * M + threadIdx.x];
      l_own = l_own * alpha_own + sum;
    }
    // O += P . C for this warp's columns
#pragma unroll
    for (int ks = 0; ks < kMmaKeys / 16; ++ks) {
      uint32_t a[MT][4];
#pragma unroll
      for (int mt = 0; mt < MT; ++mt)
        ldsm4(a[mt], Ps + (16 * mt + (lane & 7) + 8 * ((lane >> 3) & 1)) * kMmaPStride + 16 * ks + 8 * (lane >> 4));
#pragma unroll
      for (int pr = 0; pr < NT / 2; ++pr) {
        const int n0 = (warp * NT + 2 * pr) * 8;
        if (n0 < R) {
          uint32_t b[4];
          ldsm4t(b, Kt + (16 * ks + (lane & 7) + 8 * ((lane >> 3) & 1)) * DkP + n0 + 8 * (lane >> 4));
#pragma unroll
          for (int mt = 0; mt < MT; ++mt) {
            mma16816(o[mt][2 * pr], a[mt], b[0], b[1]);
            mma16816(o[mt][2 * pr + 1], a[mt], b[2], b[3]);
          }
        }
      }
    }
    __syncthreads();
  }

  if ((int)threadIdx.x < M) {
    row_top[threadIdx.x] = m_own;
    row_alpha[threadIdx.x] = l_own;
  }
  __syncthreads();
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const int r = 16 * mt + g + 8 * j;
      if (r >= valid) continue;
      const int tok = tok0 + (r0 + r) / H, h = (r0 + r) % H;
      const float m_fin = row_top[r], l_fin = row_alpha[r];
      if (n_splits > 1) {
        float* dst = part + ((size_t)((tok - first_token) * H + h) * n_splits + split) * (R + 2);
        if (warp == 0 && tq == 0) { dst[0] = m_fin; dst[1] = l_fin; }
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          const int c = (warp * NT + nt) * 8 + 2 * tq;
          if (c < R) { dst[2 + c] = o[mt][nt][2 * j]; dst[3 + c] = o[mt][nt][2 * j + 1]; }
        }
      } else {
        const float f = finish_factor(m_fin, l_fin, sink, h,
                                      gate ? __bfloat162float(gate[(size_t)tok * gate_ld + h]) : 0.f, gate != nullptr);
        __nv_bfloat16* dst = out + ((size_t)tok * H + h) * R;
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          const int c = (warp * NT + nt) * 8 + 2 * tq;
          if (c < R) *reinterpret_cast<__nv_bfloat162*>(dst + c) = __floats2bfloat162_rn(o[mt][nt][2 * j] * f, o[mt][nt][2 * j + 1] * f);
        }
      }
    }
}
#endif  // ERB_ELEM == 1

template <int NI>
void launch_attention(dim3 grid, cudaStream_t stream, const float* q_lat, const elem_t* pages, const int* block_tables,
                      int max_pages, const int* seq_of_token, const int* positions, const elem_t* gate, int gate_ld,
                      const float* sink, elem_t* out, float* part, int first_token, int n_rows, int H, int R, int Dk,
                      int page_size, int split_keys, int n_splits, float scale, int window) {
  launch_chained(latent_attention_kernel<elem_t, NI>, grid, dim3(kLatWarps * 32), 0, stream, q_lat, pages, block_tables,
                 max_pages, seq_of_token, positions, gate, gate_ld, sink, out, part, first_token, n_rows, H, R, Dk, page_size,
                 split_keys, n_splits, scale, window);
}

}  // namespace

// The token's cache row from its down-projection (when off_kv >= 0) and its query latent (when q_rank > 0).
ERB_EXPORT int erb_latent_store(const void* proj, int n_tokens, int ld, int off_kv, int R, int dr, const float* kv_weight,
                                float eps, const int* positions, const float* inv_freq, int rot_dims, const int* slots,
                                void* pages, int off_q, int q_rank, const float* q_weight, void* q_latent, void* stream) {
  if (n_tokens <= 0) return ERB_OK;
  if (off_kv >= 0 && (R <= 0 || dr < 0 || dr % 2 || rot_dims > dr || rot_dims % 2 || !kv_weight || !slots || !pages ||
                      (rot_dims > 0 && !inv_freq)))
    return fail(ERB_ERR_ARG, "latent_store: bad sizes or missing tensors for the cache row");
  if (q_rank > 0 && (!q_weight || !q_latent)) return fail(ERB_ERR_ARG, "latent_store: the query latent needs a weight and a target");
  launch_chained(latent_store_kernel<elem_t>, dim3(n_tokens), dim3(128), 0, (cudaStream_t)stream, (const elem_t*)proj, ld,
                 off_kv, R, dr, kv_weight, eps, positions, inv_freq, rot_dims, slots, (elem_t*)pages, off_q, q_rank, q_weight,
                 (elem_t*)q_latent);
  return check_launch("latent_store");
}

ERB_EXPORT int erb_latent_q_rotate(const void* q, int n_tokens, int ld, int H, int dn, int dr, int R, const int* positions,
                                   const float* inv_freq, int rot_dims, float* q_lat, void* stream) {
  if (n_tokens <= 0 || dr == 0) return ERB_OK;
  if (dr % 2 || rot_dims > dr || rot_dims % 2 || (rot_dims > 0 && !inv_freq))
    return fail(ERB_ERR_ARG, "latent_q_rotate: the rotated part must be even and at least as wide as the rotation");
  launch_chained(latent_q_rotate_kernel<elem_t>, dim3(n_tokens), dim3(128), 0, (cudaStream_t)stream, (const elem_t*)q, ld, H, dn,
                 dr, R, positions, inv_freq, rot_dims, q_lat);
  return check_launch("latent_q_rotate");
}

// Rows first_token .. first_token + n_tokens of the batch.  n_splits == 1: every row walks all its keys
// and writes its result; n_splits > 1: keys are cut at multiples of split_keys, `part` (float,
// n_tokens * H * n_splits * (R + 2)) takes the states and a second kernel merges them.
ERB_EXPORT int erb_latent_attention(const float* q_lat, const void* pages, const int* block_tables, int max_pages,
                                    const int* seq_of_token, const int* positions, const void* gate, int gate_ld,
                                    const float* sink, void* out, float* part, int first_token, int n_tokens, int H, int R,
                                    int dr, int page_size, int split_keys, int n_splits, float scale, int window,
                                    void* stream) {
  if (n_tokens <= 0) return ERB_OK;
  if (window < 0) return fail(ERB_ERR_ARG, "latent_attention: a window is 0 (none) or positive");
  const int Dk = R + dr;
  if (H <= 0 || R <= 0 || R % 2 || dr % 2 || page_size <= 0 || n_splits < 1 || n_splits > kCombineSplits ||
      (n_splits > 1 && (!part || split_keys <= 0)))
    return fail(ERB_ERR_ARG, "latent_attention: bad sizes (latent and rotated widths must be even, at most %d splits)", kCombineSplits);
  if (Dk > 1024) return fail(ERB_ERR_UNSUPPORTED, "latent_attention: cache rows of %d entries (at most 1024)", Dk);
  const int n_rows = n_tokens * H;
  const dim3 grid((n_rows + kLatWarps - 1) / kLatWarps, n_splits);
  cudaStream_t st = (cudaStream_t)stream;
#define ERB_LAT(NI) launch_attention<NI>(grid, st, q_lat, (const elem_t*)pages, block_tables, max_pages, seq_of_token, positions, \
    (const elem_t*)gate, gate_ld, sink, (elem_t*)out, part, first_token, n_rows, H, R, Dk, page_size, split_keys, n_splits, scale, window)
  if (Dk <= 128) ERB_LAT(2);
  else if (Dk <= 256) ERB_LAT(4);
  else if (Dk <= 384) ERB_LAT(6);
  else if (Dk <= 640) ERB_LAT(10);
  else ERB_LAT(16);
#undef ERB_LAT
  int rc = check_launch("latent_attention");
  if (rc || n_splits == 1) return rc;
  launch_chained(latent_combine_kernel<elem_t>, dim3(n_rows, (R + 127) / 128), dim3(128), 0, st, (const float*)part, (const elem_t*)gate, gate_ld,
                 sink, (elem_t*)out, first_token, H, R, n_splits);
  return check_launch("latent_combine");
}

// The tensor-core form (bfloat16 build only): sequences seq0 .. seq0 + n_seqs of the batch, whose rows are
// tokens seq_starts[s] .. seq_starts[s + 1]; `n_tiles` = sum over them of ceil(tokens * H / (16 * mt)).
// Needs cache rows and latents of a multiple of 8 entries (16-byte copies, whole column tiles), R <= 512.
ERB_EXPORT int erb_latent_attention_mma(const float* q_lat, const void* pages, const int* block_tables, int max_pages,
                                        const int* seq_starts, const int* positions, const void* gate, int gate_ld,
                                        const float* sink, void* out, float* part, int first_token, int seq0, int n_seqs,
                                        int n_tiles, int mt, int H, int R, int dr, int page_size, int split_keys,
                                        int n_splits, float scale, int window, void* stream) {
#if ERB_ELEM == 1
  if (n_seqs <= 0 || n_tiles <= 0) return ERB_OK;
  if (window < 0) return fail(ERB_ERR_ARG, "latent_attention_mma: a window is 0 (none) or positive");
  const int Dk = R + dr;
  if (H <= 0 || R <= 0 || R % 8 || Dk % 8 || R > 512 || page_size <= 0 || n_splits < 1 || (mt != 1 && mt != 2) ||
      ((uintptr_t)pages & 15) || (n_splits > 1 && (!part || split_keys <= 0 || split_keys % kMmaKeys)))
    return fail(ERB_ERR_UNSUPPORTED, "latent_attention_mma: sizes (latent %d, row %d) or alignment not supported", R, Dk);
  const int D16 = (Dk + 15) & ~15, DkP = D16 + 8, M = 16 * mt;
  const size_t smem = sizeof(__nv_bfloat16) * ((size_t)M * DkP + 2 * kMmaKeys * DkP + M * kMmaPStride) +
                      sizeof(float) * (2 * kMmaKeyGroups * M + 2 * M);
  if (smem > 227 * 1024) return fail(ERB_ERR_UNSUPPORTED, "latent_attention_mma: rows of %d entries need %zu bytes", Dk, smem);
  const int warps = mt == 2 ? 16 : 8;            // two row tiles: sixteen warps, two per group of keys
  const int nt = (R / 8 + warps - 1) / warps;
  const dim3 grid(n_tiles, n_splits);
  cudaStream_t st = (cudaStream_t)stream;
#define ERB_LAT_MMA(MT_, NT_, W_)                                                                                         \
  do {                                                                                                                    \
    auto kern = latent_attention_mma_kernel<MT_, NT_, W_>;                                                                \
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);                   \
    if (e != cudaSuccess) return fail(ERB_ERR_CUDA, "latent_attention_mma: %s", cudaGetErrorString(e));                   \
    launch_chained(kern, grid, dim3(W_ * 32), smem, st, q_lat, (const __nv_bfloat16*)pages, block_tables, max_pages,      \
                   seq_starts, positions, (const __nv_bfloat16*)gate, gate_ld, sink, (__nv_bfloat16*)out, part, first_token, \
                   seq0, n_seqs, H, R, Dk, page_size, split_keys, n_splits, scale, window);                               \
  } while (0)
  if (mt == 1) { if (nt <= 2) ERB_LAT_MMA(1, 2, 8); else if (nt <= 4) ERB_LAT_MMA(1, 4, 8); else ERB_LAT_MMA(1, 8, 8); }
  else { if (nt <= 2) ERB_LAT_MMA(2, 2, 16); else ERB_LAT_MMA(2, 4, 16); }
#undef ERB_LAT_MMA
  return check_launch("latent_attention_mma");
#else
  return fail(ERB_ERR_UNSUPPORTED, "latent_attention_mma: built for bfloat16 only");
#endif
}

// Merge of the splits that the tensor-core form left for `n_tokens` tokens from `first_token` on.
ERB_EXPORT int erb_latent_combine(const float* part, const void* gate, int gate_ld, const float* sink, void* out,
                                  int first_token, int n_tokens, int H, int R, int n_splits, void* stream) {
  if (n_tokens <= 0) return ERB_OK;
  if (n_splits < 1 || n_splits > kCombineSplits) return fail(ERB_ERR_ARG, "latent_combine: 1 to %d splits", kCombineSplits);
  launch_chained(latent_combine_kernel<elem_t>, dim3(n_tokens * H, (R + 127) / 128), dim3(128), 0, (cudaStream_t)stream, part, (const elem_t*)gate,
                 gate_ld, sink, (elem_t*)out, first_token, H, R, n_splits);
  return check_launch("latent_combine");
}
