// Differential attention over cache pages: every head has two score maps over the same values, and the head's output
// is the first map's result minus lambda times the second's, brought to unit RMS.
//
//   prepare:   from a token's row of the fused q/k/v product: an optional short causal convolution over time on every
//              channel (the inputs before a portion come from the request's state record), the halves of the first
//              `rot_dims` entries of each map of each q and k head turned by position * inv_freq, q written back as rows,
//              k and v written to the token's cache slot.  Everything between the product and the stores is float.
//   attention: one warp per (token, head[, split of the keys]).  A lane owns a key of every group of 32: both maps'
//              scores (scaled, soft-capped with cap * tanh(s / cap) where a cap is given), masked by the window and the
//              token's own position; the warp keeps one running maximum and denominator per map and two float accumulators
//              over the value row, of which a lane owns the columns 2 (lane + 32 i), 2 (lane + 32 i) + 1.
//              o = acc1 / l1 - lambda acc2 / l2;  out = o * rsqrt(mean(o^2) + eps) * out_scale.
//   combine:   where the keys were cut into splits (single tokens with long windows), the splits' states are merged in
//              split order and finished the same way.
//
// Cache layout (one layer): k_pages[page][kv head][offset][2 dim] holds both maps' keys of a kv head side by side,
// v_pages[page][kv head][offset][vdim] the values; token p of a sequence lives in page block_table[seq][p / page_size]
// at offset p % page_size.  Query head h reads kv head h / (H / G).  A query at position p sees the keys
// first_visible_key(p, window) .. p.  Splits lie at multiples of `split_keys`, counted from the one that holds the
// first visible key, so a token's sums do not depend on what else is in the step.
#include <algorithm>

#include "common.cuh"

using namespace erb;

ERB_DEFINE_LAST_ERROR(erb_last_error)

namespace {

template <typename T> struct Vec;  // 16-byte vectors
template <> struct Vec<float> { static constexpr int N = 4; };
template <> struct Vec<__nv_bfloat16> { static constexpr int N = 8; };
__device__ __forceinline__ void load_vec(const float* p, float* out) { load4(p, out); }
__device__ __forceinline__ void load_vec(const __nv_bfloat16* p, float* out) { load8(p, out); }

__device__ __forceinline__ float2 load_pair(const float* p) { return *reinterpret_cast<const float2*>(p); }
__device__ __forceinline__ float2 load_pair(const __nv_bfloat16* p) {
  return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p));
}

// ---------------------------------------------------------------------------------------------
// prepare.  Row layout of `proj`: H heads of [map 1 | map 2] queries (dim each), G heads of [map 1 | map 2] keys, G heads
// of values (vdim).  conv_w: float [channels][taps] in that order, or null.  conv_state: float [slots][taps - 1][channels],
// oldest first.  A "unit" is one map of a q or k head, or one value head: a warp takes a unit at a time (convolution into
// its strip of shared memory, then rotation and store), so nothing waits on the block; the block's cosines and sines of
// position * inv_freq are made once.  grid (tokens, blocks that share a token's units).
// ---------------------------------------------------------------------------------------------
constexpr int kPrepWarps = 8;

template <typename T>
__global__ void __launch_bounds__(kPrepWarps * 32)
diff_prepare_kernel(const T* __restrict__ proj, int ld, const float* __restrict__ conv_w, int taps,
                    const float* __restrict__ conv_state, const int* __restrict__ seq_of_token,
                    const int* __restrict__ seq_starts, const int* __restrict__ state_slots, const int* __restrict__ positions,
                    const float* __restrict__ inv_freq, int rot_dims, int H, int G, int dim, int vdim,
                    T* __restrict__ q_out, const int* __restrict__ slots, T* __restrict__ k_pages, T* __restrict__ v_pages,
                    int page_size) {
  chain_wait();
  extern __shared__ float prep_s[];                // [rot_dims] cosines then sines, then a strip of max(dim, vdim) per warp
  const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int half = rot_dims / 2, wide = dim > vdim ? dim : vdim;
  float* cs_s = prep_s;
  float* sn_s = prep_s + half;
  float* strip = prep_s + rot_dims + warp * wide;
  const float pos = (float)positions[t];
  for (int j = threadIdx.x; j < half; j += blockDim.x) sincosf(pos * inv_freq[j], &sn_s[j], &cs_s[j]);
  __syncthreads();
  const int qw = H * 2 * dim, kw = G * 2 * dim, channels = qw + kw + G * vdim;
  const int n_maps = 2 * (H + G), n_units = n_maps + G;
  const bool conv = conv_w && taps > 1;
  int start = 0, i = 0;
  const float* old = nullptr;
  if (conv) {
    const int seq = seq_of_token[t];
    start = seq_starts[seq];
    i = t - start;                                 // index of the token inside its portion
    old = conv_state + (size_t)state_slots[seq] * (taps - 1) * channels;
  }
  const int slot = slots ? slots[t] : -1;
  const int page = slot >= 0 ? slot / page_size : 0, offset = slot >= 0 ? slot % page_size : 0;
  for (int u = blockIdx.y * kPrepWarps + warp; u < n_units; u += gridDim.y * kPrepWarps) {
    const bool is_map = u < n_maps;
    const int width = is_map ? dim : vdim;
    const int ch0 = is_map ? u * dim : n_maps * dim + (u - n_maps) * vdim;
    if (!is_map && slot < 0) continue;             // (values only go to the cache)
    for (int e = lane; e < width; e += 32) {
      const int ch = ch0 + e;
      float acc;
      if (conv) {
        acc = 0.f;
        for (int j = 0; j < taps; ++j) {
          const int r = i - (taps - 1 - j);        // index inside the portion of the input under tap j
          const float x = r >= 0 ? Elem<T>::load(proj + (size_t)(start + r) * ld + ch) : old[(size_t)(taps - 1 + r) * channels + ch];
          acc = fmaf(conv_w[(size_t)ch * taps + j], x, acc);
        }
      } else {
        acc = (conv_w ? conv_w[ch] : 1.f) * Elem<T>::load(proj + (size_t)t * ld + ch);
      }
      strip[e] = acc;
    }
    __syncwarp();
    if (is_map) {
      const bool is_q = u < 2 * H;
      T* dst = is_q ? q_out + (size_t)t * qw + ch0
                    : k_pages + (((size_t)page * G + (u - 2 * H) / 2) * page_size + offset) * (2 * dim) + ((u - 2 * H) & 1) * dim;
      if (is_q || slot >= 0) {
        for (int e = lane; e < dim; e += 32) {
          float v = strip[e];
          if (e < half) v = strip[e] * cs_s[e] - strip[e + half] * sn_s[e];
          else if (e < rot_dims) v = strip[e] * cs_s[e - half] + strip[e - half] * sn_s[e - half];
          Elem<T>::store(dst + e, v);
        }
      }
    } else {
      T* dst = v_pages + (((size_t)page * G + (u - n_maps)) * page_size + offset) * vdim;
      for (int e = lane; e < vdim; e += 32) Elem<T>::store(dst + e, strip[e]);
    }
    __syncwarp();
  }
}

// ---------------------------------------------------------------------------------------------
// attention
// ---------------------------------------------------------------------------------------------
constexpr int kWarps = 4;          // (token, head) rows per block: neighbouring heads of a token share its keys in L1

__device__ __forceinline__ float soft_cap(float s, float cap) { return cap > 0.f ? cap * tanhf(s / cap) : s; }

// Both maps' scores of one key row (2 dim entries) against the scaled queries in shared memory.
template <typename T>
__device__ __forceinline__ void two_scores(const float* q_s, const T* key, int dim, bool vec, float& s1, float& s2) {
  constexpr int N = Vec<T>::N;
  float a = 0.f, b = 0.f;
  if (vec) {
    for (int d0 = 0; d0 < dim; d0 += N) {
      float k1[N], k2[N];
      load_vec(key + d0, k1);
      load_vec(key + dim + d0, k2);
#pragma unroll
      for (int i = 0; i < N; ++i) {
        a = fmaf(q_s[d0 + i], k1[i], a);
        b = fmaf(q_s[dim + d0 + i], k2[i], b);
      }
    }
  } else {
    for (int d = 0; d < dim; ++d) {
      a = fmaf(q_s[d], Elem<T>::load(key + d), a);
      b = fmaf(q_s[dim + d], Elem<T>::load(key + dim + d), b);
    }
  }
  s1 = a; s2 = b;
}

// The head's output from both maps' normalised sums: the difference, unit RMS over the vdim columns, a constant.
template <int VI>
__device__ __forceinline__ void finish_head(float2 (&a1)[VI], const float2 (&a2)[VI], float lambda, int vdim, float eps,
                                            float out_scale) {
  const int lane = threadIdx.x & 31;
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < VI; ++i) {
    const int c = 2 * (lane + 32 * i);
    a1[i].x -= lambda * a2[i].x;
    a1[i].y -= lambda * a2[i].y;
    if (c < vdim) ss = fmaf(a1[i].x, a1[i].x, ss);
    if (c + 1 < vdim) ss = fmaf(a1[i].y, a1[i].y, ss);
  }
  const float f = rsqrtf(warp_sum(ss) / (float)vdim + eps) * out_scale;
#pragma unroll
  for (int i = 0; i < VI; ++i) { a1[i].x *= f; a1[i].y *= f; }
}

template <typename T, int VI>
__device__ __forceinline__ void store_head(T* o, const float2 (&a)[VI], int vdim) {
  const int lane = threadIdx.x & 31;
#pragma unroll
  for (int i = 0; i < VI; ++i) {
    const int c = 2 * (lane + 32 * i);
    if (c < vdim) Elem<T>::store(o + c, a[i].x);
    if (c + 1 < vdim) Elem<T>::store(o + c + 1, a[i].y);
  }
}

// part: per (row, split) 4 floats (m1, l1, m2, l2), then the two accumulators of `vpad` floats each.
template <typename T, int VI>
__global__ void __launch_bounds__(kWarps * 32)
diff_attention_kernel(const T* __restrict__ q, const T* __restrict__ k_pages, const T* __restrict__ v_pages,
                      const int* __restrict__ block_tables, int max_pages, const int* __restrict__ seq_of_token,
                      const int* __restrict__ positions, T* __restrict__ out, float* __restrict__ part, int first_token,
                      int n_rows, int H, int G, int dim, int vdim, int page_size, int window, int split_keys, int n_splits,
                      float scale, float cap, float lambda, float eps, float out_scale) {
  chain_wait();
  extern __shared__ float q_all[];                 // [kWarps][2 dim]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row = blockIdx.x * kWarps + warp;
  if (row >= n_rows) return;                       // warps are independent: no block-wide barrier below
  const int split = blockIdx.y;
  const int t = first_token + row / H, h = row % H, g = h / (H / G);
  float* q_s = q_all + warp * 2 * dim;
  const T* q_row = q + ((size_t)t * H + h) * 2 * dim;
  for (int d = lane; d < 2 * dim; d += 32) q_s[d] = Elem<T>::load(q_row + d) * scale;
  __syncwarp();
  const int seq = seq_of_token[t], pos = positions[t];
  const int lo = first_visible_key(pos, window);
  const int base = n_splits > 1 ? (lo / split_keys + split) * split_keys : 0;
  const int begin = n_splits > 1 ? max(lo, base) : lo;
  const int end = n_splits > 1 ? min(pos + 1, base + split_keys) : pos + 1;
  const int* bt = block_tables + (size_t)seq * max_pages;
  constexpr int N = Vec<T>::N;
  const bool k_vec = dim % N == 0 && ((uintptr_t)k_pages & 15) == 0;
  const bool v_pairs = vdim % 2 == 0 && ((uintptr_t)v_pages & 7) == 0;

  float m1 = -INFINITY, m2 = -INFINITY, l1 = 0.f, l2 = 0.f;
  float2 acc1[VI], acc2[VI];
#pragma unroll
  for (int i = 0; i < VI; ++i) acc1[i] = acc2[i] = make_float2(0.f, 0.f);

  for (int k0 = begin; k0 < end; k0 += 32) {
    const int key = k0 + lane;
    const bool real = key < end;
    int kv_row = 0;                                 // (page * G + g) * page_size + offset: the key's row in both pools
    float s1 = -INFINITY, s2 = -INFINITY;
    if (real) {
      kv_row = (bt[key / page_size] * G + g) * page_size + key % page_size;
      two_scores<T>(q_s, k_pages + (size_t)kv_row * 2 * dim, dim, k_vec, s1, s2);
      s1 = soft_cap(s1, cap);
      s2 = soft_cap(s2, cap);
    }
    const float top1 = fmaxf(m1, warp_max(s1)), top2 = fmaxf(m2, warp_max(s2));
    const float alpha1 = m1 == -INFINITY ? 0.f : expf(m1 - top1), alpha2 = m2 == -INFINITY ? 0.f : expf(m2 - top2);
    const float p1 = real ? expf(s1 - top1) : 0.f, p2 = real ? expf(s2 - top2) : 0.f;
    l1 = l1 * alpha1 + warp_sum(p1);
    l2 = l2 * alpha2 + warp_sum(p2);
    m1 = top1; m2 = top2;
#pragma unroll
    for (int i = 0; i < VI; ++i) {
      acc1[i].x *= alpha1; acc1[i].y *= alpha1;
      acc2[i].x *= alpha2; acc2[i].y *= alpha2;
    }
    const int n_here = min(32, end - k0);
#pragma unroll 4
    for (int j = 0; j < n_here; ++j) {
      const float w1 = __shfl_sync(0xffffffffu, p1, j), w2 = __shfl_sync(0xffffffffu, p2, j);
      const T* v = v_pages + (size_t)__shfl_sync(0xffffffffu, kv_row, j) * vdim;
#pragma unroll
      for (int i = 0; i < VI; ++i) {
        const int c = 2 * (lane + 32 * i);
        float2 vv = make_float2(0.f, 0.f);
        if (v_pairs) {
          if (c < vdim) vv = load_pair(v + c);
        } else {
          if (c < vdim) vv.x = Elem<T>::load(v + c);
          if (c + 1 < vdim) vv.y = Elem<T>::load(v + c + 1);
        }
        acc1[i].x = fmaf(w1, vv.x, acc1[i].x); acc1[i].y = fmaf(w1, vv.y, acc1[i].y);
        acc2[i].x = fmaf(w2, vv.x, acc2[i].x); acc2[i].y = fmaf(w2, vv.y, acc2[i].y);
      }
    }
  }
  if (n_splits > 1) {
    const int vpad = 64 * VI;
    float* dst = part + ((size_t)row * n_splits + split) * (4 + 2 * vpad);
    if (lane == 0) { dst[0] = m1; dst[1] = l1; dst[2] = m2; dst[3] = l2; }
#pragma unroll
    for (int i = 0; i < VI; ++i) {
      const int c = 2 * (lane + 32 * i);
      *reinterpret_cast<float2*>(dst + 4 + c) = acc1[i];
      *reinterpret_cast<float2*>(dst + 4 + vpad + c) = acc2[i];
    }
    return;
  }
  const float r1 = 1.f / l1, r2 = 1.f / l2;
#pragma unroll
  for (int i = 0; i < VI; ++i) {
    acc1[i].x *= r1; acc1[i].y *= r1;
    acc2[i].x *= r2; acc2[i].y *= r2;
  }
  finish_head<VI>(acc1, acc2, lambda, vdim, eps, out_scale);
  store_head<T, VI>(out + ((size_t)t * H + h) * vdim, acc1, vdim);
}

// One warp per (token, head): the splits' states merged in split order (a split the row does not reach has l = 0).
template <typename T, int VI>
__global__ void __launch_bounds__(kWarps * 32)
diff_combine_kernel(const float* __restrict__ part, T* __restrict__ out, int first_token, int n_rows, int H, int vdim,
                    int n_splits, float lambda, float eps, float out_scale) {
  chain_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row = blockIdx.x * kWarps + warp;
  if (row >= n_rows) return;
  constexpr int vpad = 64 * VI, stride = 4 + 2 * vpad;
  const float* src = part + (size_t)row * n_splits * stride;
  float m1 = -INFINITY, m2 = -INFINITY;
  for (int s = 0; s < n_splits; ++s) {
    m1 = fmaxf(m1, src[s * stride]);
    m2 = fmaxf(m2, src[s * stride + 2]);
  }
  float l1 = 0.f, l2 = 0.f;
  float2 a1[VI], a2[VI];
#pragma unroll
  for (int i = 0; i < VI; ++i) a1[i] = a2[i] = make_float2(0.f, 0.f);
  for (int s = 0; s < n_splits; ++s) {
    const float* p = src + s * stride;
    const float w1 = p[0] == -INFINITY ? 0.f : expf(p[0] - m1), w2 = p[2] == -INFINITY ? 0.f : expf(p[2] - m2);
    l1 = fmaf(p[1], w1, l1);
    l2 = fmaf(p[3], w2, l2);
#pragma unroll
    for (int i = 0; i < VI; ++i) {
      const int c = 2 * (lane + 32 * i);
      const float2 x1 = *reinterpret_cast<const float2*>(p + 4 + c), x2 = *reinterpret_cast<const float2*>(p + 4 + vpad + c);
      a1[i].x = fmaf(x1.x, w1, a1[i].x); a1[i].y = fmaf(x1.y, w1, a1[i].y);
      a2[i].x = fmaf(x2.x, w2, a2[i].x); a2[i].y = fmaf(x2.y, w2, a2[i].y);
    }
  }
  const float r1 = 1.f / l1, r2 = 1.f / l2;
#pragma unroll
  for (int i = 0; i < VI; ++i) {
    a1[i].x *= r1; a1[i].y *= r1;
    a2[i].x *= r2; a2[i].y *= r2;
  }
  finish_head<VI>(a1, a2, lambda, vdim, eps, out_scale);
  const int t = first_token + row / H, h = row % H;
  store_head<T, VI>(out + ((size_t)t * H + h) * vdim, a1, vdim);
}

#if ERB_ELEM == 1
// ---------------------------------------------------------------------------------------------
// The same attention on tensor cores (bfloat16).  A block owns 64 neighbouring rows of one sequence and one kv head, a
// row being a (token, query head of that kv head) pair with the heads running fastest: the heads of a group meet their
// keys and values once.  Warp w owns 16 of the rows.  A portion of a prompt fills the tiles; a single token brings H / G
// rows, and its keys may be cut into splits (grid z) whose states a second kernel merges.  Keys and values arrive in tiles of 64 keys by 16-byte asynchronous
// copies straight from the pages into one of two stages of shared memory (rows past the end are filled with zeros).  Per
// tile and map: S = Q_m K_m^T by mma.sync m16n8k16 (queries and keys by ldmatrix, float accumulation), then scale, cap and
// mask in float, the running maximum and the weights exp(s - max) per row in float, the weights rounded to bfloat16 as
// the A operand of  O_m += P_m V  (values by ldmatrix.trans from the same stage: both maps read one value tile).  The
// epilogue is that of the general kernel, per row inside a quad of lanes.
// VT: pairs of 8-column tiles of the value row a warp accumulates (vdim <= 16 VT).
// ---------------------------------------------------------------------------------------------
constexpr int kMmaRows = 64, kMmaKeys = 64, kMmaWarps = 4;

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
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// cap * tanh(s / cap) with tanh(x) = 1 - 2 / (exp(2x) + 1) from the fast exponential and reciprocal: the absolute error of
// the capped score stays near 1e-6 cap, far below what the bfloat16 operands of the score leave.  `cap2` = 2 / cap.
__device__ __forceinline__ float soft_cap_fast(float s, float cap, float cap2) {
  return cap > 0.f ? cap - 2.f * cap * __fdividef(1.f, __expf(s * cap2) + 1.f) : s;
}

// DEC: the tile has at most 16 rows (a single token's heads of one kv head).  All warps then work on rows 0 .. 15 and share
// out a tile's keys (warp w takes keys 16 w .. 16 w + 15), each with a softmax state of its own; the four states are merged
// through shared memory at the end.  Otherwise warp w owns rows 16 w .. 16 w + 15 and walks all keys of a tile.
template <int VT, bool DEC>
__global__ void __launch_bounds__(kMmaWarps * 32)
diff_attention_mma_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k_pages,
                          const __nv_bfloat16* __restrict__ v_pages, const int* __restrict__ block_tables, int max_pages,
                          const int* __restrict__ seq_starts, const int* __restrict__ positions, __nv_bfloat16* __restrict__ out,
                          float* __restrict__ part, int first_token, int seq0, int n_seqs, int H, int G, int dim, int vdim,
                          int page_size, int window, int split_keys, int n_splits, float scale, float cap, float lambda,
                          float eps, float out_scale) {
  chain_wait();
  constexpr int kRows = DEC ? 16 : kMmaRows;        // rows of the block's tile
  constexpr int NTW = DEC ? 2 : 8;                   // 8-key tiles of a 64-key tile that one warp makes scores for
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int kw = 2 * dim, kst = kw + 8, vst = 16 * VT + 8;         // row strides in elements (16 bytes of padding)
  __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(smem_raw);  // [kRows][kst]
  __nv_bfloat16* Ks = Qs + kRows * kst;                            // [2][64][kst]
  __nv_bfloat16* Vs = Ks + 2 * kMmaKeys * kst;                     // [2][64][vst]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, tq = lane & 3;
  const int kvh = blockIdx.y, rep = H / G, split = blockIdx.z;
  const int row0_w = DEC ? 0 : 16 * warp, key0_w = DEC ? 16 * warp : 0;

  // which sequence, which of its row tiles: a sequence's rows are its (token, head of this kv head) pairs, heads fastest
  int tile = blockIdx.x, s = seq0, rows_s = 0;
  for (;; ++s) {
    if (s >= seq0 + n_seqs) return;
    rows_s = (seq_starts[s + 1] - seq_starts[s]) * rep;
    const int tiles = (rows_s + kRows - 1) / kRows;
    if (tile < tiles) break;
    tile -= tiles;
  }
  const int tok_s = seq_starts[s], r0 = tile * kRows;
  const int valid = min(kRows, rows_s - r0);
  auto token_of = [&](int r) { return tok_s + (r0 + r) / rep; };
  auto head_of = [&](int r) { return kvh * rep + (r0 + r) % rep; };
  const int pos_first = positions[token_of(0)], pos_last = positions[token_of(valid - 1)];
  // a window moves the first key; splits stay at multiples of their size, counted from the one that holds it
  const int lo = first_visible_key(pos_first, window);
  const int base = n_splits > 1 ? (lo / split_keys + split) * split_keys : 0;
  const int begin = n_splits > 1 ? max(lo, base) : lo;
  const int end = n_splits > 1 ? min(pos_last + 1, base + split_keys) : pos_last + 1;
  const int* bt = block_tables + (size_t)s * max_pages;

  // queries of the tile (rows past the valid ones: zeros)
  const int q_chunks = kw / 8;
  for (int idx = threadIdx.x; idx < kRows * q_chunks; idx += blockDim.x) {
    const int r = idx / q_chunks, c = idx % q_chunks;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (r < valid) v = *reinterpret_cast<const uint4*>(q + ((size_t)token_of(r) * H + head_of(r)) * kw + 8 * c);
    *reinterpret_cast<uint4*>(Qs + r * kst + 8 * c) = v;
  }
  if (16 * VT > vdim) {          // the copies never touch these columns of the value stages
    const int extra = 16 * VT - vdim;
    for (int idx = threadIdx.x; idx < 2 * kMmaKeys * extra; idx += blockDim.x)
      Vs[(idx / extra) * vst + vdim + idx % extra] = __float2bfloat16_rn(0.f);
  }
  // A tile's rows are shared out by warp (rows warp, warp + 4, ...).  Lane j looks up the page of the warp's j-th row, so
  // that the sixteen lookups are in flight together; then the lanes copy a row's 16-byte pieces, keys and values side by side.
  const int v_chunks = vdim / 8, kv_chunks = q_chunks + v_chunks;
  auto load_tile = [&](int k0, int stage) {
    __nv_bfloat16* kd = Ks + stage * kMmaKeys * kst;
    __nv_bfloat16* vd = Vs + stage * kMmaKeys * vst;
    const int my_key = k0 + warp + kMmaWarps * (lane & 15);
    int my_row = -1;                                             // (page * G + kv head) * page_size + offset, or -1 past the end
    if (my_key < end) my_row = (bt[my_key / page_size] * G + kvh) * page_size + my_key % page_size;
    for (int c0 = 0; c0 < kv_chunks; c0 += 32) {                 // (one turn where a row of keys and values has 32 pieces at most)
      const int c = c0 + lane;
      const bool mine = c < kv_chunks, is_k = c < q_chunks;     // (every lane takes part in the shuffles below)
      const int cc = is_k ? c : (mine ? c - q_chunks : 0);
      const __nv_bfloat16* src = (is_k ? k_pages : v_pages) + 8 * cc;
      const size_t src_ld = is_k ? kw : vdim;
      __nv_bfloat16* dst = (is_k ? kd : vd) + 8 * cc + warp * (is_k ? kst : vst);
      const int dst_ld = kMmaWarps * (is_k ? kst : vst);
#pragma unroll 4
      for (int j = 0; j < kMmaKeys / kMmaWarps; ++j) {
        const int row = __shfl_sync(0xffffffffu, my_row, j);
        if (mine) copy16(dst + j * dst_ld, src + (row >= 0 ? row : 0) * src_ld, row >= 0);
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };

  const int r_lo = row0_w + g, r_hi = r_lo + 8;                     // this thread's two rows of the tile
  const int pos_lo = r_lo < valid ? positions[token_of(r_lo)] : -1, pos_hi = r_hi < valid ? positions[token_of(r_hi)] : -1;
  const int low_lo = first_visible_key(pos_lo, window), low_hi = first_visible_key(pos_hi, window);
  // what the warp's rows see at most and at least: a tile of keys inside [w_low_max, w_pos_min] needs no mask
  const int w_last = min(valid - 1, row0_w + 15);
  const int w_pos_max = row0_w < valid ? positions[token_of(w_last)] : -1, w_pos_min = row0_w < valid ? positions[token_of(row0_w)] : -1;
  const int w_low_min = first_visible_key(w_pos_min, window), w_low_max = first_visible_key(w_pos_max, window);
  const float cap2 = cap > 0.f ? 2.f / cap : 0.f;
  float m[2][2], l[2][2];                                           // [map][row]: running maximum, this thread's share of the sum
  float o[2][2 * VT][4];
#pragma unroll
  for (int mp = 0; mp < 2; ++mp) {
    m[mp][0] = m[mp][1] = -INFINITY;
    l[mp][0] = l[mp][1] = 0.f;
#pragma unroll
    for (int nt = 0; nt < 2 * VT; ++nt)
#pragma unroll
      for (int i = 0; i < 4; ++i) o[mp][nt][i] = 0.f;
  }

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
    const __nv_bfloat16* Kt = Ks + stage * kMmaKeys * kst;
    const __nv_bfloat16* Vt = Vs + stage * kMmaKeys * vst;
    const int kf = k0 + key0_w, kl = kf + 8 * NTW - 1;              // the first and last key this warp looks at in the tile
    // (a warp whose rows all lie before its first key, or whose windows all lie behind its last, has nothing here)
    const bool idle = row0_w >= valid || kf > w_pos_max || kl < w_low_min || kf >= end;
    // no key of it is masked for any valid row (rows past the valid ones hold queries of zeros and are never stored)
    const bool plain = kf >= w_low_max && kl <= w_pos_min && kl < end;
    if (!idle) {
#pragma unroll
      for (int mp = 0; mp < 2; ++mp) {
        float sc[NTW][4];
#pragma unroll
        for (int nt = 0; nt < NTW; ++nt)
#pragma unroll
          for (int i = 0; i < 4; ++i) sc[nt][i] = 0.f;
        const __nv_bfloat16* qa = Qs + (row0_w + (lane & 7) + 8 * ((lane >> 3) & 1)) * kst + mp * dim + 8 * (lane >> 4);
        for (int kk = 0; kk < dim; kk += 16) {
          uint32_t a[4];
          ldsm4(a, qa + kk);
#pragma unroll
          for (int np = 0; np < NTW / 2; ++np) {      // a pair of 8-key tiles per ldmatrix: 16 keys, k kk .. kk + 15
            uint32_t b[4];
            ldsm4(b, Kt + (key0_w + 16 * np + (lane & 7) + 8 * (lane >> 4)) * kst + mp * dim + kk + 8 * ((lane >> 3) & 1));
            mma16816(sc[2 * np], a, b[0], b[1]);
            mma16816(sc[2 * np + 1], a, b[2], b[3]);
          }
        }
        // scale, cap, mask; the rows' maxima
        float top[2] = {m[mp][0], m[mp][1]};
        if (plain) {
#pragma unroll
          for (int nt = 0; nt < NTW; ++nt)
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const float v = soft_cap_fast(sc[nt][i] * scale, cap, cap2);
              sc[nt][i] = v;
              top[i >> 1] = fmaxf(top[i >> 1], v);
            }
        } else {
#pragma unroll
          for (int nt = 0; nt < NTW; ++nt)
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const int key = kf + 8 * nt + 2 * tq + (i & 1);
              const int row_pos = i < 2 ? pos_lo : pos_hi, row_low = i < 2 ? low_lo : low_hi;
              float v = soft_cap_fast(sc[nt][i] * scale, cap, cap2);
              if (key > row_pos || key < row_low || key >= end) v = -INFINITY;
              sc[nt][i] = v;
              top[i >> 1] = fmaxf(top[i >> 1], v);
            }
        }
#pragma unroll
        for (int r = 0; r < 2; ++r) {
          top[r] = fmaxf(top[r], __shfl_xor_sync(0xffffffffu, top[r], 1));
          top[r] = fmaxf(top[r], __shfl_xor_sync(0xffffffffu, top[r], 2));
        }
        float alpha[2], shift[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
          alpha[r] = (top[r] == -INFINITY || m[mp][r] == -INFINITY) ? (top[r] == -INFINITY ? 1.f : 0.f) : __expf(m[mp][r] - top[r]);
          shift[r] = top[r] == -INFINITY ? 0.f : top[r];             // (exp(-inf - 0) = 0 for a row that has seen no key yet)
          m[mp][r] = top[r];
          l[mp][r] *= alpha[r];
        }
        uint32_t pa[NTW / 2][4];               // the weights as A operands: [k-step of 16 keys][fragment]
#pragma unroll
        for (int nt = 0; nt < NTW; ++nt) {
          float p[4];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            p[i] = __expf(sc[nt][i] - shift[i >> 1]);
            l[mp][i >> 1] += p[i];
          }
          pa[nt >> 1][2 * (nt & 1)] = pack_bf16(p[0], p[1]);
          pa[nt >> 1][2 * (nt & 1) + 1] = pack_bf16(p[2], p[3]);
        }
        if (alpha[0] != 1.f || alpha[1] != 1.f) {       // (a tile that raised neither row's maximum rescales nothing)
#pragma unroll
          for (int nt = 0; nt < 2 * VT; ++nt) {
            o[mp][nt][0] *= alpha[0]; o[mp][nt][1] *= alpha[0];
            o[mp][nt][2] *= alpha[1]; o[mp][nt][3] *= alpha[1];
          }
        }
#pragma unroll
        for (int ks = 0; ks < NTW / 2; ++ks) {
#pragma unroll
          for (int pr = 0; pr < VT; ++pr) {
            uint32_t b[4];
            ldsm4t(b, Vt + (key0_w + 16 * ks + (lane & 7) + 8 * ((lane >> 3) & 1)) * vst + 16 * pr + 8 * (lane >> 4));
            mma16816(o[mp][2 * pr], pa[ks], b[0], b[1]);
            mma16816(o[mp][2 * pr + 1], pa[ks], b[2], b[3]);
          }
        }
      }
    }
    __syncthreads();
  }

  // each row's sums live in a quad of lanes
#pragma unroll
  for (int mp = 0; mp < 2; ++mp)
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      l[mp][r] += __shfl_xor_sync(0xffffffffu, l[mp][r], 1);
      l[mp][r] += __shfl_xor_sync(0xffffffffu, l[mp][r], 2);
    }
  const int vpad = 64 * (vdim <= 64 ? 1 : (vdim <= 128 ? 2 : 4));   // (the layout of the general kernel's split states)
  if constexpr (DEC) {
    // The warps' states of the 16 rows go to shared memory (over the stages: every warp has left the loop), float
    // [warp][map][row][16 VT + 2] with the maximum and the sum behind a row; then warp w finishes rows w, w + 4, ...
    const int mst = 16 * VT + 2;
    float* M = reinterpret_cast<float*>(smem_raw);
    __syncthreads();             // (a block without a tile of keys has not met since it wrote the queries)
#pragma unroll
    for (int mp = 0; mp < 2; ++mp)
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        if (g + 8 * r >= valid) continue;
        float* dst = M + ((size_t)(warp * 2 + mp) * 16 + g + 8 * r) * mst;
#pragma unroll
        for (int nt = 0; nt < 2 * VT; ++nt) {
          dst[8 * nt + 2 * tq] = o[mp][nt][2 * r];
          dst[8 * nt + 2 * tq + 1] = o[mp][nt][2 * r + 1];
        }
        if (tq == 0) { dst[16 * VT] = m[mp][r]; dst[16 * VT + 1] = l[mp][r]; }
      }
    __syncthreads();
    for (int row = warp; row < valid; row += kMmaWarps) {
      float wgt[2][kMmaWarps], top[2], sum[2];
#pragma unroll
      for (int mp = 0; mp < 2; ++mp) {
        top[mp] = -INFINITY;
#pragma unroll
        for (int w = 0; w < kMmaWarps; ++w) top[mp] = fmaxf(top[mp], M[((size_t)(w * 2 + mp) * 16 + row) * mst + 16 * VT]);
        sum[mp] = 0.f;
#pragma unroll
        for (int w = 0; w < kMmaWarps; ++w) {
          const float* src = M + ((size_t)(w * 2 + mp) * 16 + row) * mst + 16 * VT;
          wgt[mp][w] = src[0] == -INFINITY ? 0.f : __expf(src[0] - top[mp]);
          sum[mp] = fmaf(src[1], wgt[mp][w], sum[mp]);
        }
      }
      float acc[2][(16 * VT + 31) / 32];
#pragma unroll
      for (int mp = 0; mp < 2; ++mp)
#pragma unroll
        for (int i = 0; i < (16 * VT + 31) / 32; ++i) {
          const int c = lane + 32 * i;
          float v = 0.f;
          if (c < 16 * VT) {
#pragma unroll
            for (int w = 0; w < kMmaWarps; ++w) v = fmaf(M[((size_t)(w * 2 + mp) * 16 + row) * mst + c], wgt[mp][w], v);
          }
          acc[mp][i] = v;
        }
      const int tok = token_of(row), head = head_of(row);
      if (n_splits > 1) {
        float* dst = part + ((size_t)((tok - first_token) * H + head) * n_splits + split) * (4 + 2 * vpad);
        if (lane == 0) { dst[0] = top[0]; dst[1] = sum[0]; dst[2] = top[1]; dst[3] = sum[1]; }
#pragma unroll
        for (int i = 0; i < (16 * VT + 31) / 32; ++i) {
          const int c = lane + 32 * i;
          if (c < vdim) { dst[4 + c] = acc[0][i]; dst[4 + vpad + c] = acc[1][i]; }
        }
        continue;
      }
      const float r1 = 1.f / sum[0], r2 = lambda / sum[1];
      float ss = 0.f;
#pragma unroll
      for (int i = 0; i < (16 * VT + 31) / 32; ++i) {
        acc[0][i] = acc[0][i] * r1 - acc[1][i] * r2;
        if (lane + 32 * i < vdim) ss = fmaf(acc[0][i], acc[0][i], ss);
      }
      const float f = rsqrtf(warp_sum(ss) / (float)vdim + eps) * out_scale;
      __nv_bfloat16* dst = out + ((size_t)tok * H + head) * vdim;
#pragma unroll
      for (int i = 0; i < (16 * VT + 31) / 32; ++i) {
        const int c = lane + 32 * i;
        if (c < vdim) dst[c] = __float2bfloat16_rn(acc[0][i] * f);
      }
    }
    return;
  }
  if (n_splits > 1) {          // the states of this split
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const int row = r ? r_hi : r_lo;
      if (row >= valid) continue;
      float* dst = part + ((size_t)((token_of(row) - first_token) * H + head_of(row)) * n_splits + split) * (4 + 2 * vpad);
      if (tq == 0) { dst[0] = m[0][r]; dst[1] = l[0][r]; dst[2] = m[1][r]; dst[3] = l[1][r]; }
#pragma unroll
      for (int nt = 0; nt < 2 * VT; ++nt) {
        const int c = 8 * nt + 2 * tq;
        if (c < vdim) {
          *reinterpret_cast<float2*>(dst + 4 + c) = make_float2(o[0][nt][2 * r], o[0][nt][2 * r + 1]);
          *reinterpret_cast<float2*>(dst + 4 + vpad + c) = make_float2(o[1][nt][2 * r], o[1][nt][2 * r + 1]);
        }
      }
    }
    return;
  }
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const float r1 = 1.f / l[0][r], r2 = lambda / l[1][r];
    float ss = 0.f;
#pragma unroll
    for (int nt = 0; nt < 2 * VT; ++nt)
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const float v = o[0][nt][2 * r + i] * r1 - o[1][nt][2 * r + i] * r2;
        o[0][nt][2 * r + i] = v;
        if (8 * nt + 2 * tq + i < vdim) ss = fmaf(v, v, ss);
      }
    ss += __shfl_xor_sync(0xffffffffu, ss, 1);
    ss += __shfl_xor_sync(0xffffffffu, ss, 2);
    const float f = rsqrtf(ss / (float)vdim + eps) * out_scale;
    const int row = r ? r_hi : r_lo;
    if (row < valid) {
      __nv_bfloat16* dst = out + ((size_t)token_of(row) * H + head_of(row)) * vdim;
#pragma unroll
      for (int nt = 0; nt < 2 * VT; ++nt) {
        const int c = 8 * nt + 2 * tq;
        if (c < vdim) *reinterpret_cast<__nv_bfloat162*>(dst + c) = __floats2bfloat162_rn(o[0][nt][2 * r] * f, o[0][nt][2 * r + 1] * f);
      }
    }
  }
}

// Single tokens whose kv head serves at most 8 query heads: both maps in ONE tile of 16 rows.  Row r < 8 holds head r's
// first map as [q1 | 0], row 8 + r its second map as [0 | q2], so one product over the whole key row [k1 | k2] gives both
// maps' scores, one softmax state a row serves both, and one accumulator holds a1 in rows 0 .. 7 and a2 in rows 8 .. 15: half
// the registers, products and exponentials of the two-pass form.  The four warps share out a tile's keys; their states are
// merged through shared memory; splits over grid z.  One block per (sequence, kv head, split).
template <int VT>
__global__ void __launch_bounds__(kMmaWarps * 32, 3)
diff_attention_mma_packed_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k_pages,
                                 const __nv_bfloat16* __restrict__ v_pages, const int* __restrict__ block_tables, int max_pages,
                                 const int* __restrict__ seq_starts, const int* __restrict__ positions,
                                 __nv_bfloat16* __restrict__ out, float* __restrict__ part, int first_token, int seq0, int H, int G,
                                 int dim, int vdim, int page_size, int window, int split_keys, int n_splits, float scale, float cap,
                                 float lambda, float eps, float out_scale) {
  chain_wait();
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int kw = 2 * dim, kst = kw + 8, vst = 16 * VT + 8;
  __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(smem_raw);  // [16][kst]
  __nv_bfloat16* Ks = Qs + 16 * kst;                               // [2][64][kst]
  __nv_bfloat16* Vs = Ks + 2 * kMmaKeys * kst;                     // [2][64][vst]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, tq = lane & 3;
  const int s = seq0 + blockIdx.x, kvh = blockIdx.y, rep = H / G, split = blockIdx.z;
  const int tok = seq_starts[s], pos = positions[tok];
  const int lo = first_visible_key(pos, window);
  const int base = n_splits > 1 ? (lo / split_keys + split) * split_keys : 0;
  const int begin = n_splits > 1 ? max(lo, base) : lo;
  const int end = n_splits > 1 ? min(pos + 1, base + split_keys) : pos + 1;
  const int* bt = block_tables + (size_t)s * max_pages;
  const int key0_w = 16 * warp;

  const int q_chunks = kw / 8, half_chunks = dim / 8;
  for (int idx = threadIdx.x; idx < 16 * q_chunks; idx += blockDim.x) {
    const int r = idx / q_chunks, c = idx % q_chunks;
    const int head = r & 7, second = r >> 3;                       // rows 0 .. 7: first maps, 8 .. 15: second maps
    uint4 v = make_uint4(0, 0, 0, 0);
    if (head < rep && (c >= half_chunks) == (second != 0))
      v = *reinterpret_cast<const uint4*>(q + ((size_t)tok * H + kvh * rep + head) * kw + 8 * c);
    *reinterpret_cast<uint4*>(Qs + r * kst + 8 * c) = v;
  }
  if (16 * VT > vdim) {
    const int extra = 16 * VT - vdim;
    for (int idx = threadIdx.x; idx < 2 * kMmaKeys * extra; idx += blockDim.x)
      Vs[(idx / extra) * vst + vdim + idx % extra] = __float2bfloat16_rn(0.f);
  }
  const int v_chunks = vdim / 8, kv_chunks = q_chunks + v_chunks;
  auto load_tile = [&](int k0, int stage) {
    __nv_bfloat16* kd = Ks + stage * kMmaKeys * kst;
    __nv_bfloat16* vd = Vs + stage * kMmaKeys * vst;
    const int my_key = k0 + warp + kMmaWarps * (lane & 15);
    int my_row = -1;
    if (my_key < end) my_row = (bt[my_key / page_size] * G + kvh) * page_size + my_key % page_size;
    for (int c0 = 0; c0 < kv_chunks; c0 += 32) {
      const int c = c0 + lane;
      const bool mine = c < kv_chunks, is_k = c < q_chunks;
      const int cc = is_k ? c : (mine ? c - q_chunks : 0);
      const __nv_bfloat16* src = (is_k ? k_pages : v_pages) + 8 * cc;
      const size_t src_ld = is_k ? kw : vdim;
      __nv_bfloat16* dst = (is_k ? kd : vd) + 8 * cc + warp * (is_k ? kst : vst);
      const int dst_ld = kMmaWarps * (is_k ? kst : vst);
#pragma unroll 4
      for (int j = 0; j < kMmaKeys / kMmaWarps; ++j) {
        const int row = __shfl_sync(0xffffffffu, my_row, j);
        if (mine) copy16(dst + j * dst_ld, src + (row >= 0 ? row : 0) * src_ld, row >= 0);
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };

  const float cap2 = cap > 0.f ? 2.f / cap : 0.f;
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};          // rows g (a first map) and g + 8 (a second map)
  float o[2 * VT][4];
#pragma unroll
  for (int nt = 0; nt < 2 * VT; ++nt)
#pragma unroll
    for (int i = 0; i < 4; ++i) o[nt][i] = 0.f;

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
    const __nv_bfloat16* Kt = Ks + stage * kMmaKeys * kst;
    const __nv_bfloat16* Vt = Vs + stage * kMmaKeys * vst;
    const int kf = k0 + key0_w, kl = kf + 15;
    if (kf < end) {                                                // (keys begin .. end - 1 are all inside the window and not after the token)
      float sc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
      const __nv_bfloat16* qa = Qs + ((lane & 7) + 8 * ((lane >> 3) & 1)) * kst + 8 * (lane >> 4);
      const __nv_bfloat16* kb = Kt + (key0_w + (lane & 7) + 8 * (lane >> 4)) * kst + 8 * ((lane >> 3) & 1);
      for (int kk = 0; kk < kw; kk += 16) {
        uint32_t a[4], b[4];
        ldsm4(a, qa + kk);
        ldsm4(b, kb + kk);
        mma16816(sc[0], a, b[0], b[1]);
        mma16816(sc[1], a, b[2], b[3]);
      }
      float top[2] = {m[0], m[1]};
#pragma unroll
      for (int nt = 0; nt < 2; ++nt)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          float v = soft_cap_fast(sc[nt][i] * scale, cap, cap2);
          if (kl >= end && kf + 8 * nt + 2 * tq + (i & 1) >= end) v = -INFINITY;
          sc[nt][i] = v;
          top[i >> 1] = fmaxf(top[i >> 1], v);
        }
      float alpha[2], shift[2];
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        top[r] = fmaxf(top[r], __shfl_xor_sync(0xffffffffu, top[r], 1));
        top[r] = fmaxf(top[r], __shfl_xor_sync(0xffffffffu, top[r], 2));
        alpha[r] = m[r] == -INFINITY ? 0.f : __expf(m[r] - top[r]);
        shift[r] = top[r];                                          // (finite: the warp has at least one key here)
        m[r] = top[r];
        l[r] *= alpha[r];
      }
      uint32_t pa[4];
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
        float p[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          p[i] = __expf(sc[nt][i] - shift[i >> 1]);
          l[i >> 1] += p[i];
        }
        pa[2 * nt] = pack_bf16(p[0], p[1]);
        pa[2 * nt + 1] = pack_bf16(p[2], p[3]);
      }
      if (alpha[0] != 1.f || alpha[1] != 1.f) {
#pragma unroll
        for (int nt = 0; nt < 2 * VT; ++nt) {
          o[nt][0] *= alpha[0]; o[nt][1] *= alpha[0];
          o[nt][2] *= alpha[1]; o[nt][3] *= alpha[1];
        }
      }
#pragma unroll
      for (int pr = 0; pr < VT; ++pr) {
        uint32_t b[4];
        ldsm4t(b, Vt + (key0_w + (lane & 7) + 8 * ((lane >> 3) & 1)) * vst + 16 * pr + 8 * (lane >> 4));
        mma16816(o[2 * pr], pa, b[0], b[1]);
        mma16816(o[2 * pr + 1], pa, b[2], b[3]);
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l[r] += __shfl_xor_sync(0xffffffffu, l[r], 1);
    l[r] += __shfl_xor_sync(0xffffffffu, l[r], 2);
  }
  // the warps' states to shared memory (over the stages), float [warp][row 16][16 VT + 2]; then warp w finishes heads w, w + 4
  const int mst = 16 * VT + 2;
  float* M = reinterpret_cast<float*>(smem_raw);
  __syncthreads();
  if (g < rep) {
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      float* dst = M + ((size_t)warp * 16 + g + 8 * r) * mst;
#pragma unroll
      for (int nt = 0; nt < 2 * VT; ++nt) {
        dst[8 * nt + 2 * tq] = o[nt][2 * r];
        dst[8 * nt + 2 * tq + 1] = o[nt][2 * r + 1];
      }
      if (tq == 0) { dst[16 * VT] = m[r]; dst[16 * VT + 1] = l[r]; }
    }
  }
  __syncthreads();
  const int vpad = 64 * (vdim <= 64 ? 1 : (vdim <= 128 ? 2 : 4));
  for (int head = warp; head < rep; head += kMmaWarps) {
    float wgt[2][kMmaWarps], top[2], sum[2];
#pragma unroll
    for (int mp = 0; mp < 2; ++mp) {
      const int row = head + 8 * mp;
      top[mp] = -INFINITY;
#pragma unroll
      for (int w = 0; w < kMmaWarps; ++w) top[mp] = fmaxf(top[mp], M[((size_t)w * 16 + row) * mst + 16 * VT]);
      sum[mp] = 0.f;
#pragma unroll
      for (int w = 0; w < kMmaWarps; ++w) {
        const float* src = M + ((size_t)w * 16 + row) * mst + 16 * VT;
        wgt[mp][w] = src[0] == -INFINITY ? 0.f : __expf(src[0] - top[mp]);
        sum[mp] = fmaf(src[1], wgt[mp][w], sum[mp]);
      }
    }
    float acc[2][(16 * VT + 31) / 32];
#pragma unroll
    for (int mp = 0; mp < 2; ++mp)
#pragma unroll
      for (int i = 0; i < (16 * VT + 31) / 32; ++i) {
        const int c = lane + 32 * i;
        float v = 0.f;
        if (c < 16 * VT) {
#pragma unroll
          for (int w = 0; w < kMmaWarps; ++w) v = fmaf(M[((size_t)w * 16 + head + 8 * mp) * mst + c], wgt[mp][w], v);
        }
        acc[mp][i] = v;
      }
    const int qh = kvh * rep + head;
    if (n_splits > 1) {
      float* dst = part + ((size_t)((tok - first_token) * H + qh) * n_splits + split) * (4 + 2 * vpad);
      if (lane == 0) { dst[0] = top[0]; dst[1] = sum[0]; dst[2] = top[1]; dst[3] = sum[1]; }
#pragma unroll
      for (int i = 0; i < (16 * VT + 31) / 32; ++i) {
        const int c = lane + 32 * i;
        if (c < vdim) { dst[4 + c] = acc[0][i]; dst[4 + vpad + c] = acc[1][i]; }
      }
      continue;
    }
    const float r1 = 1.f / sum[0], r2 = lambda / sum[1];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < (16 * VT + 31) / 32; ++i) {
      acc[0][i] = acc[0][i] * r1 - acc[1][i] * r2;
      if (lane + 32 * i < vdim) ss = fmaf(acc[0][i], acc[0][i], ss);
    }
    const float f = rsqrtf(warp_sum(ss) / (float)vdim + eps) * out_scale;
    __nv_bfloat16* dst = out + ((size_t)tok * H + qh) * vdim;
#pragma unroll
    for (int i = 0; i < (16 * VT + 31) / 32; ++i) {
      const int c = lane + 32 * i;
      if (c < vdim) dst[c] = __float2bfloat16_rn(acc[0][i] * f);
    }
  }
}

template <int VT>
int launch_mma_packed(cudaStream_t st, const void* q, const void* k_pages, const void* v_pages, const int* block_tables,
                      int max_pages, const int* seq_starts, const int* positions, void* out, float* part, int first_token,
                      int n_tokens, int seq0, int n_seqs, int H, int G, int dim, int vdim, int page_size, int window, int split_keys,
                      int n_splits, float scale, float cap, float lambda, float eps, float out_scale) {
  size_t smem = sizeof(__nv_bfloat16) * ((size_t)(16 + 2 * kMmaKeys) * (2 * dim + 8) + 2 * (size_t)kMmaKeys * (16 * VT + 8));
  smem = std::max(smem, sizeof(float) * kMmaWarps * 16 * (size_t)(16 * VT + 2));
  auto kern = diff_attention_mma_packed_kernel<VT>;
  if (smem > 227 * 1024) return fail(ERB_ERR_UNSUPPORTED, "diff_attention_mma: maps of %d entries need %zu bytes of shared memory", dim, smem);
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return fail(ERB_ERR_CUDA, "diff_attention_mma: %s", cudaGetErrorString(e));
  }
  launch_chained(kern, dim3(n_seqs, G, n_splits), dim3(kMmaWarps * 32), smem, st, (const __nv_bfloat16*)q,
                 (const __nv_bfloat16*)k_pages, (const __nv_bfloat16*)v_pages, block_tables, max_pages, seq_starts, positions,
                 (__nv_bfloat16*)out, part, first_token, seq0, H, G, dim, vdim, page_size, window, split_keys, n_splits, scale, cap,
                 lambda, eps, out_scale);
  int rc = check_launch("diff_attention_mma");
  if (rc || n_splits == 1) return rc;
  const int n_rows = n_tokens * H;
  auto merge = [&](auto kernel) {
    launch_chained(kernel, dim3((n_rows + kWarps - 1) / kWarps), dim3(kWarps * 32), 0, st, (const float*)part, (__nv_bfloat16*)out,
                   first_token, n_rows, H, vdim, n_splits, lambda, eps, out_scale);
  };
  if (vdim <= 64) merge(diff_combine_kernel<__nv_bfloat16, 1>); else merge(diff_combine_kernel<__nv_bfloat16, 2>);
  return check_launch("diff_combine");
}

template <int VT, bool DEC>
int launch_mma(cudaStream_t st, const void* q, const void* k_pages, const void* v_pages, const int* block_tables, int max_pages,
               const int* seq_starts, const int* positions, void* out, float* part, int first_token, int n_tokens, int seq0,
               int n_seqs, int n_tiles, int H, int G, int dim, int vdim, int page_size, int window, int split_keys, int n_splits,
               float scale, float cap, float lambda, float eps, float out_scale) {
  const int rows = DEC ? 16 : kMmaRows;
  size_t smem = sizeof(__nv_bfloat16) * ((size_t)(rows + 2 * kMmaKeys) * (2 * dim + 8) + 2 * (size_t)kMmaKeys * (16 * VT + 8));
  if (DEC) smem = std::max(smem, sizeof(float) * kMmaWarps * 2 * 16 * (size_t)(16 * VT + 2));     // (the merge of the warps' states)
  auto kern = diff_attention_mma_kernel<VT, DEC>;
  if (smem > 227 * 1024) return fail(ERB_ERR_UNSUPPORTED, "diff_attention_mma: maps of %d entries need %zu bytes of shared memory", dim, smem);
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return fail(ERB_ERR_CUDA, "diff_attention_mma: %s", cudaGetErrorString(e));
  }
  launch_chained(kern, dim3(n_tiles, G, n_splits), dim3(kMmaWarps * 32), smem, st, (const __nv_bfloat16*)q,
                 (const __nv_bfloat16*)k_pages, (const __nv_bfloat16*)v_pages, block_tables, max_pages, seq_starts, positions,
                 (__nv_bfloat16*)out, part, first_token, seq0, n_seqs, H, G, dim, vdim, page_size, window, split_keys, n_splits, scale,
                 cap, lambda, eps, out_scale);
  int rc = check_launch("diff_attention_mma");
  if (rc || n_splits == 1) return rc;
  const int n_rows = n_tokens * H;
  auto merge = [&](auto kernel) {
    launch_chained(kernel, dim3((n_rows + kWarps - 1) / kWarps), dim3(kWarps * 32), 0, st, (const float*)part, (__nv_bfloat16*)out,
                   first_token, n_rows, H, vdim, n_splits, lambda, eps, out_scale);
  };
  if (vdim <= 64) merge(diff_combine_kernel<__nv_bfloat16, 1>); else merge(diff_combine_kernel<__nv_bfloat16, 2>);
  return check_launch("diff_combine");
}
#endif  // ERB_ELEM == 1

template <int VI>
int launch_attention(cudaStream_t st, const elem_t* q, const elem_t* k_pages, const elem_t* v_pages, const int* block_tables,
                     int max_pages, const int* seq_of_token, const int* positions, elem_t* out, float* part, int first_token,
                     int n_rows, int H, int G, int dim, int vdim, int page_size, int window, int split_keys, int n_splits,
                     float scale, float cap, float lambda, float eps, float out_scale) {
  const size_t smem = sizeof(float) * kWarps * 2 * dim;
  auto kern = diff_attention_kernel<elem_t, VI>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return fail(ERB_ERR_CUDA, "diff_attention: %s", cudaGetErrorString(e));
  }
  const dim3 grid((n_rows + kWarps - 1) / kWarps, n_splits);
  launch_chained(kern, grid, dim3(kWarps * 32), smem, st, q, k_pages, v_pages, block_tables, max_pages, seq_of_token, positions,
                 out, part, first_token, n_rows, H, G, dim, vdim, page_size, window, split_keys, n_splits, scale, cap, lambda, eps,
                 out_scale);
  int rc = check_launch("diff_attention");
  if (rc || n_splits == 1) return rc;
  launch_chained(diff_combine_kernel<elem_t, VI>, dim3((n_rows + kWarps - 1) / kWarps), dim3(kWarps * 32), 0, st,
                 (const float*)part, out, first_token, n_rows, H, vdim, n_splits, lambda, eps, out_scale);
  return check_launch("diff_combine");
}

}  // namespace

// Floats of scratch per (token, head, split) for value rows of `vdim` entries.
ERB_EXPORT int erb_diff_part_floats(int vdim) {
  const int vi = vdim <= 64 ? 1 : (vdim <= 128 ? 2 : 4);
  return 4 + 2 * 64 * vi;
}

ERB_EXPORT int erb_diff_prepare(const void* proj, int n_tokens, int ld, const float* conv_w, int taps, const float* conv_state,
                                const int* seq_of_token, const int* seq_starts, const int* state_slots, const int* positions,
                                const float* inv_freq, int rot_dims, int H, int G, int dim, int vdim, void* q_out,
                                const int* slots, void* k_pages, void* v_pages, int page_size, void* stream) {
  if (n_tokens <= 0) return ERB_OK;
  if (H <= 0 || G <= 0 || H % G || dim <= 0 || vdim <= 0 || rot_dims < 0 || rot_dims % 2 || rot_dims > dim ||
      (rot_dims && !inv_freq) || taps < 1 || (taps > 1 && (!conv_w || !conv_state)) || page_size <= 0)
    return fail(ERB_ERR_ARG, "diff_prepare: bad sizes (rot_dims %d of dim %d, %d taps)", rot_dims, dim, taps);
  const int channels = (H + G) * 2 * dim + G * vdim;
  if (ld < channels) return fail(ERB_ERR_ARG, "diff_prepare: rows too narrow");
  const size_t smem = sizeof(float) * ((size_t)rot_dims + (size_t)kPrepWarps * (dim > vdim ? dim : vdim));
  if (smem > 200 * 1024) return fail(ERB_ERR_UNSUPPORTED, "diff_prepare: maps of %d and values of %d entries", dim, vdim);
  // few tokens: a token's units are spread over several blocks
  const int n_units = 2 * (H + G) + G;
  const int share = n_tokens >= 256 ? 1 : (n_units + kPrepWarps - 1) / kPrepWarps;
  auto kern = diff_prepare_kernel<elem_t>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return fail(ERB_ERR_CUDA, "diff_prepare: %s", cudaGetErrorString(e));
  }
  launch_chained(kern, dim3(n_tokens, share), dim3(kPrepWarps * 32), smem, (cudaStream_t)stream, (const elem_t*)proj, ld, conv_w, taps, conv_state,
                 seq_of_token, seq_starts, state_slots, positions, inv_freq, rot_dims, H, G, dim, vdim, (elem_t*)q_out, slots,
                 (elem_t*)k_pages, (elem_t*)v_pages, page_size);
  return check_launch("diff_prepare");
}

// Rows first_token .. first_token + n_tokens of the batch.  n_splits == 1: every row walks all its keys and writes its
// result; n_splits > 1: `part` (float, n_tokens * H * n_splits * erb_diff_part_floats(vdim)) takes the splits' states
// and a second kernel merges them.
ERB_EXPORT int erb_diff_attention(const void* q, const void* k_pages, const void* v_pages, const int* block_tables, int max_pages,
                                  const int* seq_of_token, const int* positions, void* out, float* part, int first_token,
                                  int n_tokens, int H, int G, int dim, int vdim, int page_size, int window, int split_keys,
                                  int n_splits, float scale, float cap, float lambda, float eps, float out_scale, void* stream) {
  if (n_tokens <= 0) return ERB_OK;
  if (H <= 0 || G <= 0 || H % G || dim <= 0 || vdim <= 0 || vdim > 256 || page_size <= 0 || window < 0 || n_splits < 1 ||
      (n_splits > 1 && (!part || split_keys <= 0 || ((uintptr_t)part & 7))))
    return fail(ERB_ERR_ARG, "diff_attention: bad sizes (values of at most 256 entries, window >= 0)");
  cudaStream_t st = (cudaStream_t)stream;
  const int n_rows = n_tokens * H;
#define ERB_DIFF(VI) launch_attention<VI>(st, (const elem_t*)q, (const elem_t*)k_pages, (const elem_t*)v_pages, block_tables,    \
    max_pages, seq_of_token, positions, (elem_t*)out, part, first_token, n_rows, H, G, dim, vdim, page_size, window, split_keys, \
    n_splits, scale, cap, lambda, eps, out_scale)
  if (vdim <= 64) return ERB_DIFF(1);
  if (vdim <= 128) return ERB_DIFF(2);
  return ERB_DIFF(4);
#undef ERB_DIFF
}

// The tensor-core form (bfloat16 build only): sequences seq0 .. seq0 + n_seqs of the batch, whose rows are tokens
// seq_starts[s] .. seq_starts[s + 1] (tokens first_token .. first_token + n_tokens in all); `n_tiles` = sum over them of
// ceil(tokens * (H / G) / tile_rows), tile_rows 64 (portions) or 16 (single tokens: the warps share out a tile's keys);
// tile_rows 8: single tokens (one per sequence) with at most 8 heads a kv head, both maps packed into one tile of 16 rows.  With n_splits > 1 (single tokens) `part` takes the splits' states as for erb_diff_attention.
// Needs maps of a multiple of 16 entries and value rows of a multiple of 8 entries, at most 128.
ERB_EXPORT int erb_diff_attention_mma(const void* q, const void* k_pages, const void* v_pages, const int* block_tables,
                                      int max_pages, const int* seq_starts, const int* positions, void* out, float* part,
                                      int first_token, int n_tokens, int seq0, int n_seqs, int n_tiles, int tile_rows, int H, int G,
                                      int dim, int vdim, int page_size, int window, int split_keys, int n_splits, float scale,
                                      float cap, float lambda, float eps, float out_scale, void* stream) {
#if ERB_ELEM == 1
  if (n_seqs <= 0 || n_tiles <= 0) return ERB_OK;
  if (H <= 0 || G <= 0 || H % G || dim <= 0 || dim % 16 || vdim <= 0 || vdim % 8 || vdim > 128 || page_size <= 0 || window < 0 ||
      ((uintptr_t)q & 15) || ((uintptr_t)k_pages & 15) || ((uintptr_t)v_pages & 15) || ((uintptr_t)out & 3) || n_splits < 1 ||
      (n_splits > 1 && (!part || split_keys <= 0 || ((uintptr_t)part & 7))) || (tile_rows != 8 && tile_rows != 16 && tile_rows != 64) ||
      (tile_rows == 8 && (H / G > 8 || n_tiles != n_seqs || n_tokens != n_seqs)))
    return fail(ERB_ERR_UNSUPPORTED, "diff_attention_mma: sizes (maps of %d, values of %d) or alignment not supported", dim, vdim);
  cudaStream_t st = (cudaStream_t)stream;
#define ERB_DIFF_MMA(VT) (tile_rows == 8 ? launch_mma_packed<VT>(st, q, k_pages, v_pages, block_tables, max_pages, seq_starts, positions, \
    out, part, first_token, n_tokens, seq0, n_seqs, H, G, dim, vdim, page_size, window, split_keys, n_splits, scale, cap, lambda, eps,   \
    out_scale) : tile_rows == 16 ? ERB_DIFF_MMA2(VT, true) : ERB_DIFF_MMA2(VT, false))
#define ERB_DIFF_MMA2(VT, DEC) launch_mma<VT, DEC>(st, q, k_pages, v_pages, block_tables, max_pages, seq_starts, positions, out, part,         \
    first_token, n_tokens, seq0, n_seqs, n_tiles, H, G, dim, vdim, page_size, window, split_keys, n_splits, scale, cap, lambda, eps, \
    out_scale)
  if (vdim <= 32) return ERB_DIFF_MMA(2);
  if (vdim <= 64) return ERB_DIFF_MMA(4);
  if (vdim <= 96) return ERB_DIFF_MMA(6);
  return ERB_DIFF_MMA(8);
#undef ERB_DIFF_MMA
#undef ERB_DIFF_MMA2
#else
  return fail(ERB_ERR_UNSUPPORTED, "diff_attention_mma: the tensor-core form is built for bfloat16 only");
#endif
}
