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
// prepare: one block per token.  Row layout of `proj`: H heads of [map 1 | map 2] queries (dim each), G heads of
// [map 1 | map 2] keys, G heads of values (vdim).  conv_w: float [channels][taps] in that order, or null.
// conv_state: float [slots][taps - 1][channels], oldest first.
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256)
diff_prepare_kernel(const T* __restrict__ proj, int ld, const float* __restrict__ conv_w, int taps,
                    const float* __restrict__ conv_state, const int* __restrict__ seq_of_token,
                    const int* __restrict__ seq_starts, const int* __restrict__ state_slots, const int* __restrict__ positions,
                    const float* __restrict__ inv_freq, int rot_dims, int H, int G, int dim, int vdim,
                    T* __restrict__ q_out, const int* __restrict__ slots, T* __restrict__ k_pages, T* __restrict__ v_pages,
                    int page_size) {
  chain_wait();
  extern __shared__ float row_s[];                 // the token's q, k and v after the convolution
  const int t = blockIdx.x;
  const int qw = H * 2 * dim, kw = G * 2 * dim, channels = qw + kw + G * vdim;
  const T* row = proj + (size_t)t * ld;
  if (conv_w && taps > 1) {
    const int seq = seq_of_token[t], start = seq_starts[seq], i = t - start;
    const float* old = conv_state + (size_t)state_slots[seq] * (taps - 1) * channels;
    for (int ch = threadIdx.x; ch < channels; ch += blockDim.x) {
      float acc = 0.f;
      for (int j = 0; j < taps; ++j) {
        const int r = i - (taps - 1 - j);          // index inside the portion of the input under tap j
        const float u = r >= 0 ? Elem<T>::load(proj + (size_t)(start + r) * ld + ch) : old[(size_t)(taps - 1 + r) * channels + ch];
        acc = fmaf(conv_w[(size_t)ch * taps + j], u, acc);
      }
      row_s[ch] = acc;
    }
  } else {
    for (int ch = threadIdx.x; ch < channels; ch += blockDim.x) row_s[ch] = (conv_w ? conv_w[ch] : 1.f) * Elem<T>::load(row + ch);
  }
  __syncthreads();
  const float pos = (float)positions[t];
  const int half = rot_dims / 2;
  const int slot = slots ? slots[t] : -1;
  const int page = slot >= 0 ? slot / page_size : 0, offset = slot >= 0 ? slot % page_size : 0;
  // queries and keys: maps of `dim` entries, the first rot_dims of each turned in halves
  const int n_maps = 2 * (H + G);
  for (int idx = threadIdx.x; idx < n_maps * dim; idx += blockDim.x) {
    const int map = idx / dim, e = idx % dim;
    const float* m = row_s + map * dim;
    float v = m[e];
    if (e < rot_dims) {
      const int j = e < half ? e : e - half;
      float sn, cs;
      sincosf(pos * inv_freq[j], &sn, &cs);
      v = e < half ? m[e] * cs - m[e + half] * sn : m[e] * cs + m[e - half] * sn;
    }
    if (map < 2 * H) {
      Elem<T>::store(q_out + (size_t)t * qw + idx, v);
    } else if (slot >= 0) {
      const int kk = idx - qw, g = kk / (2 * dim), ee = kk % (2 * dim);
      Elem<T>::store(k_pages + (((size_t)page * G + g) * page_size + offset) * (2 * dim) + ee, v);
    }
  }
  if (slot >= 0) {
    for (int idx = threadIdx.x; idx < G * vdim; idx += blockDim.x) {
      const int g = idx / vdim, e = idx % vdim;
      Elem<T>::store(v_pages + (((size_t)page * G + g) * page_size + offset) * vdim + e, row_s[qw + kw + idx]);
    }
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
  const size_t smem = sizeof(float) * channels;
  if (smem > 200 * 1024) return fail(ERB_ERR_UNSUPPORTED, "diff_prepare: rows of %d channels", channels);
  auto kern = diff_prepare_kernel<elem_t>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return fail(ERB_ERR_CUDA, "diff_prepare: %s", cudaGetErrorString(e));
  }
  launch_chained(kern, dim3(n_tokens), dim3(256), smem, (cudaStream_t)stream, (const elem_t*)proj, ld, conv_w, taps, conv_state,
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
