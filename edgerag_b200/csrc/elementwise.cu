// Row-wise kernels of the decoder step: embedding rows, residual add + RMSNorm, rotary position
// encoding fused with the write of keys and values into cache pages, and the SwiGLU gate.
//
// The residual stream is held in 32-bit for both element types; `T` is the type of everything
// that feeds a matrix product (bfloat16 on the serving path, float on the 32-bit path).
#include "common.cuh"

using namespace erb;

ERB_DEFINE_LAST_ERROR(erb_last_error)

// ---------------------------------------------------------------------------------------------
// Embedding: hidden[t, :] = scale * table[ids[t], :]  or  scale * embeds[embed_row[t], :]   (written as float)
// An id outside [0, vocab) sets *status = 1 + t and writes zeros; nothing is read out of range.
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void embed_rows_kernel(float* __restrict__ hidden, const T* __restrict__ table,
                                  const T* __restrict__ embeds, const int* __restrict__ ids,
                                  const int* __restrict__ embed_row, int hidden_size, int vocab,
                                  int n_embed_rows, int* __restrict__ status, float scale) {
  chain_wait();
  const int t = blockIdx.x;
  const int er = embed_row ? embed_row[t] : -1;
  const T* src = nullptr;
  if (er >= 0) {
    if (er < n_embed_rows && embeds) src = embeds + (size_t)er * hidden_size;
  } else {
    const int id = ids[t];
    if (id >= 0 && id < vocab) src = table + (size_t)id * hidden_size;
  }
  if (!src && threadIdx.x == 0) atomicCAS(status, 0, 1 + t);
  float* dst = hidden + (size_t)t * hidden_size;
  for (int i = threadIdx.x; i < hidden_size; i += blockDim.x) dst[i] = src ? Elem<T>::load(src + i) * scale : 0.f;
}

ERB_EXPORT int erb_embed_rows(void* hidden, const void* table, const void* embeds, const int* ids,
                              const int* embed_row, int n_tokens, int hidden_size, int vocab,
                              int n_embed_rows, int* status, float scale, void* stream) {
  if (n_tokens <= 0) return ERB_OK;
  if (hidden_size <= 0 || vocab <= 0) return fail(ERB_ERR_ARG, "embed_rows: bad sizes");
  const int threads = hidden_size >= 1024 ? 256 : 128;
  launch_chained(embed_rows_kernel<elem_t>, dim3(n_tokens), dim3(threads), 0, (cudaStream_t)stream, (float*)hidden,
      (const elem_t*)table, (const elem_t*)embeds, ids, embed_row, hidden_size, vocab, n_embed_rows, status, scale);
  return check_launch("embed_rows");
}

// ---------------------------------------------------------------------------------------------
// Residual add + RMSNorm.
//   r = hidden[row] (+ dscale * delta[row])   in float, stored back when `write_back` (dscale: a constant of the model
//                                             that multiplies every update of its stream; 1 for most)
// The update may also come as `n_parts` float arrays of partial sums, `part_stride` floats apart (a
// product whose k was split over blocks): delta = round_T(((p0 + p1) + p2) + ...), added in float in that
// order and rounded to T once, as if the product had been stored in T like every other update.
//   y = weight * round_T( r * rsqrt(mean(r^2) + eps) )     rounded to T once more
// The statistics, the scale and the residual sum are float; the cast to T comes before the
// weight multiply, as in the reference's RMSNorm.  `rows`, when given, selects the rows of
// hidden/delta that are read (output row i comes from input row rows[i]).
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void add_rmsnorm_kernel(float* __restrict__ hidden, const T* __restrict__ delta,
                                   const float* __restrict__ parts, int n_parts, size_t part_stride,
                                   const float* __restrict__ weight, T* __restrict__ out,
                                   const int* __restrict__ rows, int hidden_size, float eps,
                                   int write_back, int exact, float dscale) {
  chain_wait();
  extern __shared__ float row_cache[];  // hidden_size floats, then 32 of scratch
  float* scratch = row_cache + hidden_size;
  const int o = blockIdx.x;
  const int r = rows ? rows[o] : o;
  float* h = hidden + (size_t)r * hidden_size;
  const T* d = delta ? delta + (size_t)r * hidden_size : nullptr;
  const float* ps = parts ? parts + (size_t)r * hidden_size : nullptr;
  float ss = 0.f;
  for (int i = threadIdx.x; i < hidden_size; i += blockDim.x) {
    float v = h[i];
    if (d) v += dscale * Elem<T>::load(d + i);
    if (ps) {
      float sum = ps[i];
      for (int sp = 1; sp < n_parts; ++sp) sum += ps[sp * part_stride + i];
      v += dscale * Elem<T>::round(sum);
    }
    row_cache[i] = v;
    if (write_back && (d || ps)) h[i] = v;
    ss += v * v;
  }
  const float total = block_sum(ss, scratch);
  const float rs = rsqrtf(total / (float)hidden_size + eps);
  T* y = out + (size_t)o * hidden_size;
  for (int i = threadIdx.x; i < hidden_size; i += blockDim.x) {
    const float normed = exact ? row_cache[i] * rs : Elem<T>::round(row_cache[i] * rs);
    Elem<T>::store(y + i, weight[i] * normed);
  }
}

// Four elements per thread and step (hidden_size a multiple of 4): 16-byte accesses to the residual.
template <typename T> struct Pack4;
template <> struct Pack4<float> {
  static __device__ __forceinline__ void load(const float* p, float* v) { load4(p, v); }
  static __device__ __forceinline__ void store(float* p, const float* v) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  }
};
template <> struct Pack4<__nv_bfloat16> {
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float* v) {
    const uint2 raw = *reinterpret_cast<const uint2*>(p);
    v[0] = __uint_as_float(raw.x << 16); v[1] = __uint_as_float(raw.x & 0xffff0000u);
    v[2] = __uint_as_float(raw.y << 16); v[3] = __uint_as_float(raw.y & 0xffff0000u);
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, const float* v) {
    __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
    *reinterpret_cast<uint2*>(p) = make_uint2(*reinterpret_cast<uint32_t*>(&a), *reinterpret_cast<uint32_t*>(&b));
  }
};

// The same with 16-byte accesses.  The order in which a row's squares are added is that of VT
// "virtual threads" (element group g of the row belongs to virtual thread g % VT; warp trees over
// 32 neighbouring virtual threads, then one tree over the warp sums), whatever the number of real
// threads: a block of VT / R threads keeps R partial sums per thread, one per virtual thread it
// stands for.  So the launch may use fewer, busier threads for many rows and more threads for the
// few rows of a decode step, and a row's result does not depend on which.
// REGS: the row fits one pass (hidden_size <= 4 * VT), so a thread keeps its elements in registers between
// the sum and the scaling instead of parking the row in shared memory; the sums are the same.
// PARTS: the update is the sum of partial sums (see above) instead of `delta`.
template <typename T, int R, bool REGS, bool PARTS = false>
__global__ void __launch_bounds__(512, ((REGS && R > 1) || PARTS) ? 2 : 4)   // (32 registers where 2,048 threads stay resident)
add_rmsnorm_vec4_kernel(float* __restrict__ hidden, const T* __restrict__ delta,
                                        const float* __restrict__ parts, int n_parts, size_t part_stride,
                                        const float* __restrict__ weight, T* __restrict__ out,
                                        const int* __restrict__ rows, int hidden_size, float eps,
                                        int write_back, int flags, float dscale) {
  extern __shared__ float row_cache[];
  const int settled = flags & 1;
  const bool exact = flags & 2;        // the normed value is not rounded before the weight multiplies it
  float* scratch = REGS ? row_cache : row_cache + hidden_size;
  float keep[REGS ? R : 1][4];
  const int o = blockIdx.x;
  const int r = rows ? rows[o] : o;            // the step's metadata: not written by the kernel before
  float* h = hidden + (size_t)r * hidden_size;
  const T* d = (!PARTS && delta) ? delta + (size_t)r * hidden_size : nullptr;
  const float* ps = PARTS ? parts + (size_t)r * hidden_size : nullptr;
  const int threads = blockDim.x, vt = threads * R;
  // the norm's weight is a constant: this thread's first four are loaded before the wait
  const int i_first = threadIdx.x * 4;
  float w_first[4] = {0.f, 0.f, 0.f, 0.f};
  if (i_first < hidden_size) load4(weight + i_first, w_first);
  // `settled`: the residual stream was last written two or more kernels ago (the kernel just before this
  // one wrote `delta` only), so its rows may be read while that kernel is still running.
  if constexpr (REGS) {
    if (settled) {
#pragma unroll
      for (int q = 0; q < R; ++q) {
        const int i = (threadIdx.x + q * threads) * 4;
        if (i < hidden_size) load4(h + i, keep[q]);
      }
    }
  }
  chain_wait();
  float ss[R];
#pragma unroll
  for (int q = 0; q < R; ++q) ss[q] = 0.f;
  for (int base = 0; base < hidden_size; base += vt * 4) {
#pragma unroll
    for (int q = 0; q < R; ++q) {
      const int i = base + (threadIdx.x + q * threads) * 4;
      if (i >= hidden_size) continue;
      float v[4];
      if (REGS && settled) {
#pragma unroll
        for (int j = 0; j < 4; ++j) v[j] = keep[q][j];
      } else {
        load4(h + i, v);
      }
      if constexpr (PARTS) {
        float dv[4];
        load4(ps + i, dv);
#pragma unroll 4
        for (int sp = 1; sp < n_parts; ++sp) {
          float pv[4];
          load4(ps + sp * part_stride + i, pv);
#pragma unroll
          for (int j = 0; j < 4; ++j) dv[j] += pv[j];
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) v[j] += dscale * Elem<T>::round(dv[j]);
        if (write_back) *reinterpret_cast<float4*>(h + i) = make_float4(v[0], v[1], v[2], v[3]);
      } else if (d) {
        float dv[4];
        Pack4<T>::load(d + i, dv);
#pragma unroll
        for (int j = 0; j < 4; ++j) v[j] += dscale * dv[j];
        if (write_back) *reinterpret_cast<float4*>(h + i) = make_float4(v[0], v[1], v[2], v[3]);
      }
      if constexpr (REGS) {
#pragma unroll
        for (int j = 0; j < 4; ++j) keep[q][j] = v[j];
      } else {
        *reinterpret_cast<float4*>(row_cache + i) = make_float4(v[0], v[1], v[2], v[3]);
      }
      ss[q] += v[0] * v[0] + v[1] * v[1] + v[2] * v[2] + v[3] * v[3];
    }
  }
  // block_sum over the virtual threads
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = threads >> 5;
#pragma unroll
  for (int q = 0; q < R; ++q) ss[q] = warp_sum(ss[q]);
  __syncthreads();
  if (lane == 0) {
#pragma unroll
    for (int q = 0; q < R; ++q) scratch[warp + q * warps] = ss[q];
  }
  __syncthreads();
  const float total = warp_sum(lane < warps * R ? scratch[lane] : 0.f);
  const float rs = rsqrtf(total / (float)hidden_size + eps);
  T* y = out + (size_t)o * hidden_size;
  if constexpr (REGS) {
#pragma unroll
    for (int q = 0; q < R; ++q) {
      const int i = (threadIdx.x + q * threads) * 4;
      if (i >= hidden_size) continue;
      float w[4], v[4];
      if (q == 0) {
#pragma unroll
        for (int j = 0; j < 4; ++j) w[j] = w_first[j];
      } else {
        load4(weight + i, w);
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) v[j] = w[j] * (exact ? keep[q][j] * rs : Elem<T>::round(keep[q][j] * rs));
      Pack4<T>::store(y + i, v);
    }
    return;
  }
  for (int i = threadIdx.x * 4; i < hidden_size; i += threads * 4) {
    float v[4], w[4];
    load4(row_cache + i, v);
    if (i == i_first) {
#pragma unroll
      for (int j = 0; j < 4; ++j) w[j] = w_first[j];
    } else {
      load4(weight + i, w);
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) v[j] = w[j] * (exact ? v[j] * rs : Elem<T>::round(v[j] * rs));
    Pack4<T>::store(y + i, v);
  }
}

namespace {
int run_add_rmsnorm(void* hidden, const void* delta, const float* parts, int n_parts, size_t part_stride,
                    const float* weight, void* out, const int* rows, int n_rows, int hidden_size, float eps,
                    int write_back, int settled, float dscale, void* stream) {
  if (n_rows <= 0) return ERB_OK;
  const size_t smem = (size_t)(hidden_size + 32) * sizeof(float);
  if (smem > 200 * 1024) return fail(ERB_ERR_UNSUPPORTED, "add_rmsnorm: hidden_size %d too large", hidden_size);
  if (rows && write_back) return fail(ERB_ERR_ARG, "add_rmsnorm: row selection cannot write back");
  // The order of a row's sum depends on the width only (this many virtual threads), whatever the batch;
  // at 2048 and more, one pass of 16-byte loads per thread (the row's latency is paid once).
  const int threads = hidden_size >= 2048 ? 512 : (hidden_size >= 512 ? 256 : 128);
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(add_rmsnorm_kernel<elem_t>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return fail(ERB_ERR_CUDA, "add_rmsnorm: %s", cudaGetErrorString(e));
  }
  const bool vec = hidden_size % 4 == 0 && !((uintptr_t)hidden & 15) && !((uintptr_t)delta & 7) &&
                   !((uintptr_t)out & 7) && !((uintptr_t)weight & 15) && !((uintptr_t)parts & 15) && part_stride % 4 == 0;
  if (vec && parts) {
    const bool one_pass = hidden_size <= threads * 4;
    const size_t small = 32 * sizeof(float);
    if (one_pass) {
      launch_chained(add_rmsnorm_vec4_kernel<elem_t, 1, true, true>, dim3(n_rows), dim3(threads), small, (cudaStream_t)stream,
          (float*)hidden, (const elem_t*)nullptr, parts, n_parts, part_stride, weight, (elem_t*)out, rows, hidden_size, eps,
          write_back, settled, dscale);
    } else {
      if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(add_rmsnorm_vec4_kernel<elem_t, 1, false, true>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return fail(ERB_ERR_CUDA, "add_rmsnorm: %s", cudaGetErrorString(e));
      }
      launch_chained(add_rmsnorm_vec4_kernel<elem_t, 1, false, true>, dim3(n_rows), dim3(threads), smem, (cudaStream_t)stream,
          (float*)hidden, (const elem_t*)nullptr, parts, n_parts, part_stride, weight, (elem_t*)out, rows, hidden_size, eps,
          write_back, settled, dscale);
    }
  } else if (vec) {
    // many rows of 2048 and more: half the threads, two virtual threads each (same sums, see the kernel)
    const bool halve = threads == 512 && n_rows > 64;
    const bool one_pass = hidden_size <= threads * 4;     // a row fits the registers of its block
    if (smem > 48 * 1024 && !one_pass) {
      cudaError_t e = halve ? cudaFuncSetAttribute(add_rmsnorm_vec4_kernel<elem_t, 2, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)
                            : cudaFuncSetAttribute(add_rmsnorm_vec4_kernel<elem_t, 1, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return fail(ERB_ERR_CUDA, "add_rmsnorm: %s", cudaGetErrorString(e));
    }
    const size_t small = 32 * sizeof(float);
    if (halve && one_pass)
      launch_chained(add_rmsnorm_vec4_kernel<elem_t, 2, true>, dim3(n_rows), dim3(256), small, (cudaStream_t)stream, (float*)hidden,
          (const elem_t*)delta, nullptr, 0, (size_t)0, weight, (elem_t*)out, rows, hidden_size, eps, write_back, settled, dscale);
    else if (halve)
      launch_chained(add_rmsnorm_vec4_kernel<elem_t, 2, false>, dim3(n_rows), dim3(256), smem, (cudaStream_t)stream, (float*)hidden,
          (const elem_t*)delta, nullptr, 0, (size_t)0, weight, (elem_t*)out, rows, hidden_size, eps, write_back, settled, dscale);
    else if (one_pass)
      launch_chained(add_rmsnorm_vec4_kernel<elem_t, 1, true>, dim3(n_rows), dim3(threads), small, (cudaStream_t)stream, (float*)hidden,
          (const elem_t*)delta, nullptr, 0, (size_t)0, weight, (elem_t*)out, rows, hidden_size, eps, write_back, settled, dscale);
    else
      launch_chained(add_rmsnorm_vec4_kernel<elem_t, 1, false>, dim3(n_rows), dim3(threads), smem, (cudaStream_t)stream, (float*)hidden,
          (const elem_t*)delta, nullptr, 0, (size_t)0, weight, (elem_t*)out, rows, hidden_size, eps, write_back, settled, dscale);
  } else {
    launch_chained(add_rmsnorm_kernel<elem_t>, dim3(n_rows), dim3(threads), smem, (cudaStream_t)stream, (float*)hidden,
        (const elem_t*)delta, parts, n_parts, part_stride, weight, (elem_t*)out, rows, hidden_size, eps, write_back, settled & 2, dscale);
  }
  return check_launch("add_rmsnorm");
}
}  // namespace

ERB_EXPORT int erb_add_rmsnorm(void* hidden, const void* delta, const float* weight, void* out,
                               const int* rows, int n_rows, int hidden_size, float eps, int write_back,
                               int settled, float delta_scale, void* stream) {
  return run_add_rmsnorm(hidden, delta, nullptr, 0, 0, weight, out, rows, n_rows, hidden_size, eps, write_back, settled, delta_scale,
                         stream);
}

// The same with the update given as `n_parts` arrays of partial sums [rows of hidden][hidden_size], float,
// `part_stride` floats from one to the next; they are added in their order.
ERB_EXPORT int erb_add_rmsnorm_parts(void* hidden, const float* parts, int n_parts, long long part_stride, const float* weight,
                                     void* out, const int* rows, int n_rows, int hidden_size, float eps, int write_back,
                                     int settled, float delta_scale, void* stream) {
  if (!parts || n_parts < 1 || part_stride < 0) return fail(ERB_ERR_ARG, "add_rmsnorm_parts: bad arguments");
  return run_add_rmsnorm(hidden, nullptr, parts, n_parts, (size_t)part_stride, weight, out, rows, n_rows, hidden_size, eps,
                         write_back, settled, delta_scale, stream);
}

// hidden[row] += delta[row] without a norm (the last residual of a stack that ends without one).
template <typename T>
__global__ void residual_add_kernel(float* __restrict__ hidden, const T* __restrict__ delta, size_t n, float dscale) {
  chain_wait();
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) hidden[i] += dscale * Elem<T>::load(delta + i);
}

// hidden += round_T(p0 + p1 + ...) for float partial sums, `part_stride` floats apart.
template <typename T>
__global__ void residual_add_parts_kernel(float* __restrict__ hidden, const float* __restrict__ parts, int n_parts,
                                          size_t part_stride, size_t n, float dscale) {
  chain_wait();
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  float sum = parts[i];
  for (int sp = 1; sp < n_parts; ++sp) sum += parts[sp * part_stride + i];
  hidden[i] += dscale * Elem<T>::round(sum);
}

ERB_EXPORT int erb_residual_add_parts(void* hidden, const float* parts, int n_parts, long long part_stride, long long n,
                                      float delta_scale, void* stream) {
  if (n <= 0) return ERB_OK;
  if (!parts || n_parts < 1 || part_stride < 0) return fail(ERB_ERR_ARG, "residual_add_parts: bad arguments");
  const int threads = 256;
  const unsigned blocks = (unsigned)((n + threads - 1) / threads);
  launch_chained(residual_add_parts_kernel<elem_t>, dim3(blocks), dim3(threads), 0, (cudaStream_t)stream, (float*)hidden, parts,
      n_parts, (size_t)part_stride, (size_t)n, delta_scale);
  return check_launch("residual_add_parts");
}

ERB_EXPORT int erb_residual_add(void* hidden, const void* delta, long long n, float delta_scale, void* stream) {
  if (n <= 0) return ERB_OK;
  const int threads = 256;
  const unsigned blocks = (unsigned)((n + threads - 1) / threads);
  launch_chained(residual_add_kernel<elem_t>, dim3(blocks), dim3(threads), 0, (cudaStream_t)stream, (float*)hidden,
      (const elem_t*)delta, (size_t)n, delta_scale);
  return check_launch("residual_add");
}

// ---------------------------------------------------------------------------------------------
// Rotary position encoding (halves convention) + cache write.
//   qkv: [n_tokens, (nq + 2 nkv) * D], rows hold q heads, then k heads, then v heads.
//   angle[j] = position * inv_freq[j] (float), j < rot_dim / 2; the pair is (x[j], x[j + rot/2]).
//   q is rotated in place.  k is rotated and, with v, written to the token's cache slot:
//   slot = page * page_size + offset (negative: the token writes nothing), page layout
//   [page][kv head][offset][D].  With `write_kv == 0` only q is rotated (the layer reads the
//   cache of another layer); with `rot_dim == 0` nothing is rotated (another position encoding
//   acted before) and the kernel is only the cache write.
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void rope_cache_write_kernel(T* __restrict__ qkv, const int* __restrict__ positions,
                                        const float* __restrict__ inv_freq, const int* __restrict__ slots,
                                        T* __restrict__ k_pages, T* __restrict__ v_pages, int nq, int nkv,
                                        int head_dim, int rot_dim, int page_size, int write_kv) {
  chain_wait();
  const int t = blockIdx.x;
  const int row_width = (nq + 2 * nkv) * head_dim;
  T* row = qkv + (size_t)t * row_width;
  const float pos = (float)positions[t];
  const int half_rot = rot_dim / 2;
  const int half_all = head_dim / 2;  // work items per head: one per pair of elements
  const int slot = (write_kv && slots) ? slots[t] : -1;
  const int page = slot >= 0 ? slot / page_size : 0;
  const int offset = slot >= 0 ? (int)(slot % page_size) : 0;

  const int rot_heads = nq + nkv;
  // q and k heads: pairs (j, j + half_rot) inside the rotated part, pass-through pairs beyond it.
  for (int w = threadIdx.x; w < rot_heads * half_all; w += blockDim.x) {
    const int head = w / half_all, j = w % half_all;
    T* x = row + (size_t)head * head_dim;
    int i0, i1;
    float o0, o1;
    if (j < half_rot) {
      i0 = j; i1 = j + half_rot;
      float sn, cs;
      sincosf(pos * inv_freq[j], &sn, &cs);
      const float a = Elem<T>::load(x + i0), b = Elem<T>::load(x + i1);
      rotate_pair(a, b, cs, sn, o0, o1);
    } else {
      i0 = rot_dim + 2 * (j - half_rot); i1 = i0 + 1;
      o0 = Elem<T>::load(x + i0); o1 = Elem<T>::load(x + i1);
    }
    if (head < nq) {
      if (j < half_rot) { Elem<T>::store(x + i0, o0); Elem<T>::store(x + i1, o1); }
    } else if (slot >= 0) {
      const int kvh = head - nq;
      T* dst = k_pages + (((size_t)page * nkv + kvh) * page_size + offset) * head_dim;
      Elem<T>::store(dst + i0, o0);
      Elem<T>::store(dst + i1, o1);
    }
  }
  if (slot >= 0) {
    const T* v = row + (size_t)(nq + nkv) * head_dim;
    for (int w = threadIdx.x; w < nkv * head_dim; w += blockDim.x) {
      const int kvh = w / head_dim, i = w % head_dim;
      v_pages[(((size_t)page * nkv + kvh) * page_size + offset) * head_dim + i] = v[w];
    }
  }
}

// Sixteen bytes of consecutive elements as floats, and back (8 bfloat16 or 4 float).
template <typename T> struct Wide;
template <> struct Wide<float> {
  static constexpr int N = 4;
  static __device__ __forceinline__ void load(const float* p, float* v) { load4(p, v); }
  static __device__ __forceinline__ void store(float* p, const float* v) { Pack4<float>::store(p, v); }
};
template <> struct Wide<__nv_bfloat16> {
  static constexpr int N = 8;
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float* v) { load8(p, v); }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, const float* v) {
    uint4 raw;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
    *reinterpret_cast<uint4*>(p) = raw;
  }
};

// Full rotation (rot_dim == head_dim, a multiple of 2 * Wide<T>::N): the angles of a token are computed
// once per block into shared memory, every work item moves sixteen bytes of each half, and the heads of
// a token are spread over gridDim.y blocks so that a few decode tokens still fill the GPU.
template <typename T>
__global__ void rope_cache_write_wide_kernel(T* __restrict__ qkv, const int* __restrict__ positions,
                                             const float* __restrict__ inv_freq, const int* __restrict__ slots,
                                             T* __restrict__ k_pages, T* __restrict__ v_pages, int nq, int nkv,
                                             int head_dim, int page_size, int write_kv) {
  constexpr int N = Wide<T>::N;
  extern __shared__ float trig[];            // cos[half], sin[half]
  const int t = blockIdx.x;
  const int half = head_dim / 2;
  const float pos = (float)positions[t];
  for (int j = threadIdx.x; j < half; j += blockDim.x) sincosf(pos * inv_freq[j], trig + half + j, trig + j);
  const int slot = (write_kv && slots) ? slots[t] : -1;
  __syncthreads();
  chain_wait();
  const int row_width = (nq + 2 * nkv) * head_dim;
  T* row = qkv + (size_t)t * row_width;
  const int page = slot >= 0 ? slot / page_size : 0;
  const int offset = slot >= 0 ? slot % page_size : 0;
  const int per_head = half / N;              // items per rotated head
  const int rot_items = (nq + nkv) * per_head;
  const int v_items = slot >= 0 ? nkv * head_dim / N : 0;
  const int stride = gridDim.y * blockDim.x;
  for (int w = blockIdx.y * blockDim.x + threadIdx.x; w < rot_items + v_items; w += stride) {
    if (w < rot_items) {
      const int head = w / per_head, j = (w % per_head) * N;
      if (head >= nq && slot < 0) continue;
      T* x = row + (size_t)head * head_dim;
      float a[N], b[N], lo[N], hi[N];
      Wide<T>::load(x + j, a);
      Wide<T>::load(x + j + half, b);
#pragma unroll
      for (int i = 0; i < N; ++i) rotate_pair(a[i], b[i], trig[j + i], trig[half + j + i], lo[i], hi[i]);
      T* dst = x;
      if (head >= nq) dst = k_pages + (((size_t)page * nkv + (head - nq)) * page_size + offset) * head_dim;
      Wide<T>::store(dst + j, lo);
      Wide<T>::store(dst + j + half, hi);
    } else {
      const int i = (w - rot_items) * N;
      const int kvh = i / head_dim, e = i % head_dim;
      float v[N];
      Wide<T>::load(row + (size_t)(nq + nkv) * head_dim + i, v);
      Wide<T>::store(v_pages + (((size_t)page * nkv + kvh) * page_size + offset) * head_dim + e, v);
    }
  }
}

// The same with eight-byte accesses (four elements), for head sizes that are a multiple of 8 only.
template <typename T>
__global__ void rope_cache_write_vec4_kernel(T* __restrict__ qkv, const int* __restrict__ positions,
                                             const float* __restrict__ inv_freq, const int* __restrict__ slots,
                                             T* __restrict__ k_pages, T* __restrict__ v_pages, int nq, int nkv,
                                             int head_dim, int page_size, int write_kv) {
  // Positions and slots are the step's metadata and the frequencies are constants: the angles are
  // ready before the kernel that produces qkv has finished.
  extern __shared__ float trig[];            // cos[half], sin[half]
  const int t = blockIdx.x;
  const int half = head_dim / 2;
  const float pos = (float)positions[t];
  for (int j = threadIdx.x; j < half; j += blockDim.x) sincosf(pos * inv_freq[j], trig + half + j, trig + j);
  const int slot = (write_kv && slots) ? slots[t] : -1;
  __syncthreads();
  chain_wait();
  const int row_width = (nq + 2 * nkv) * head_dim;
  T* row = qkv + (size_t)t * row_width;
  const int page = slot >= 0 ? slot / page_size : 0;
  const int offset = slot >= 0 ? slot % page_size : 0;
  const int per_head = half / 4;              // items per rotated head
  const int rot_items = (nq + nkv) * per_head;
  const int v_items = slot >= 0 ? nkv * head_dim / 4 : 0;
  const int stride = gridDim.y * blockDim.x;
  for (int w = blockIdx.y * blockDim.x + threadIdx.x; w < rot_items + v_items; w += stride) {
    if (w < rot_items) {
      const int head = w / per_head, j = (w % per_head) * 4;
      if (head >= nq && slot < 0) continue;
      T* x = row + (size_t)head * head_dim;
      float a[4], b[4], lo[4], hi[4];
      Pack4<T>::load(x + j, a);
      Pack4<T>::load(x + j + half, b);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        rotate_pair(a[i], b[i], trig[j + i], trig[half + j + i], lo[i], hi[i]);
      }
      T* dst = x;
      if (head >= nq) dst = k_pages + (((size_t)page * nkv + (head - nq)) * page_size + offset) * head_dim;
      Pack4<T>::store(dst + j, lo);
      Pack4<T>::store(dst + j + half, hi);
    } else {
      const int i = (w - rot_items) * 4;
      const int kvh = i / head_dim, e = i % head_dim;
      float v[4];
      Pack4<T>::load(row + (size_t)(nq + nkv) * head_dim + i, v);
      Pack4<T>::store(v_pages + (((size_t)page * nkv + kvh) * page_size + offset) * head_dim + e, v);
    }
  }
}

// Whether every row of qkv and every head inside it starts on a 16-byte boundary.
static bool row_bytes_16(int nq, int nkv, int head_dim, size_t elem) {
  return ((size_t)(nq + 2 * nkv) * head_dim * elem) % 16 == 0 && ((size_t)head_dim * elem) % 32 == 0;
}

ERB_EXPORT int erb_rope_cache_write(void* qkv, const int* positions, const float* inv_freq,
                                    const int* slots, void* k_pages, void* v_pages, int n_tokens,
                                    int nq, int nkv, int head_dim, int rot_dim, int page_size,
                                    int write_kv, void* stream) {
  if (n_tokens <= 0) return ERB_OK;
  if (head_dim <= 0 || head_dim % 2 || rot_dim < 0 || rot_dim > head_dim || rot_dim % 2)
    return fail(ERB_ERR_ARG, "rope_cache_write: head_dim %d / rot_dim %d must be even, rot <= head", head_dim, rot_dim);
  if (rot_dim > 0 && !inv_freq) return fail(ERB_ERR_ARG, "rope_cache_write: inv_freq missing");
  if (write_kv && (!slots || !k_pages || !v_pages || page_size <= 0))
    return fail(ERB_ERR_ARG, "rope_cache_write: cache arguments missing");
  const int work = (nq + nkv) * head_dim / 2;
  const int threads = work >= 512 ? 256 : 128;
  if (rot_dim == head_dim && head_dim % 8 == 0 && !((uintptr_t)qkv & 15) && !((uintptr_t)k_pages & 15) &&
      !((uintptr_t)v_pages & 15)) {
    const bool wide = head_dim % (2 * Wide<elem_t>::N) == 0 && row_bytes_16(nq, nkv, head_dim, sizeof(elem_t));
    const int per = wide ? Wide<elem_t>::N : 4;
    const int items = (nq + nkv) * head_dim / (2 * per) + nkv * head_dim / per;
    int y = (items + 127) / 128;
    const int want = (sm_count() * 8 + n_tokens - 1) / n_tokens;      // enough blocks for every SM
    if (y > want) y = want;
    if (y < 1) y = 1;
    if (wide) {
      launch_chained(rope_cache_write_wide_kernel<elem_t>, dim3(dim3(n_tokens, y)), dim3(128), head_dim * sizeof(float), (cudaStream_t)stream,
          (elem_t*)qkv, positions, inv_freq, slots, (elem_t*)k_pages, (elem_t*)v_pages, nq, nkv, head_dim, page_size, write_kv);
      return check_launch("rope_cache_write");
    }
    launch_chained(rope_cache_write_vec4_kernel<elem_t>, dim3(dim3(n_tokens, y)), dim3(128), head_dim * sizeof(float), (cudaStream_t)stream, 
        (elem_t*)qkv, positions, inv_freq, slots, (elem_t*)k_pages, (elem_t*)v_pages, nq, nkv, head_dim, page_size,
        write_kv);
    return check_launch("rope_cache_write");
  }
  launch_chained(rope_cache_write_kernel<elem_t>, dim3(n_tokens), dim3(threads), 0, (cudaStream_t)stream, (elem_t*)qkv, positions,
      inv_freq, slots, (elem_t*)k_pages, (elem_t*)v_pages, nq, nkv, head_dim, rot_dim, page_size, write_kv);
  return check_launch("rope_cache_write");
}

// ---------------------------------------------------------------------------------------------
// SwiGLU gate: out[t, i] = silu(gate_up[t, i]) * gate_up[t, I + i], computed in float.
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ gate_up, T* __restrict__ out, int inter, size_t total) {
  chain_wait();
  size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const size_t t = idx / inter;
  const int i = (int)(idx % inter);
  const T* row = gate_up + t * 2 * (size_t)inter;
  const float g = Elem<T>::load(row + i), u = Elem<T>::load(row + inter + i);
  Elem<T>::store(out + idx, silu_mul(g, u));
}

template <typename T> struct Vec16;   // 16-byte groups
template <> struct Vec16<float> {
  static constexpr int N = 4;
  static __device__ __forceinline__ void load(const float* p, float* v) { load4(p, v); }
  static __device__ __forceinline__ void store(float* p, const float* v) { Pack4<float>::store(p, v); }
};
template <> struct Vec16<__nv_bfloat16> {
  static constexpr int N = 8;
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float* v) { load8(p, v); }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, const float* v) {
    Pack4<__nv_bfloat16>::store(p, v);
    Pack4<__nv_bfloat16>::store(p + 4, v + 4);
  }
};

template <typename T>
__global__ void swiglu_vec_kernel(const T* __restrict__ gate_up, T* __restrict__ out, int inter, size_t groups) {
  chain_wait();
  constexpr int N = Vec16<T>::N;
  const size_t gidx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (gidx >= groups) return;
  const int per_row = inter / N;
  const size_t t = gidx / per_row;
  const int i = (int)(gidx % per_row) * N;
  const T* row = gate_up + t * 2 * (size_t)inter;
  float g[N], u[N];
  Vec16<T>::load(row + i, g);
  Vec16<T>::load(row + inter + i, u);
#pragma unroll
  for (int j = 0; j < N; ++j) g[j] = silu_mul(g[j], u[j]);
  Vec16<T>::store(out + t * (size_t)inter + i, g);
}

ERB_EXPORT int erb_swiglu(const void* gate_up, void* out, int n_tokens, int inter, void* stream) {
  if (n_tokens <= 0) return ERB_OK;
  if (inter <= 0) return fail(ERB_ERR_ARG, "swiglu: bad intermediate size");
  const size_t total = (size_t)n_tokens * inter;
  const int threads = 256;
  if (inter % Vec16<elem_t>::N == 0 && !((uintptr_t)gate_up & 15) && !((uintptr_t)out & 15)) {
    const size_t groups = total / Vec16<elem_t>::N;
    launch_chained(swiglu_vec_kernel<elem_t>, dim3((unsigned)((groups + threads - 1) / threads)), dim3(threads), 0, (cudaStream_t)stream, 
        (const elem_t*)gate_up, (elem_t*)out, inter, groups);
    return check_launch("swiglu");
  }
  const unsigned blocks = (unsigned)((total + threads - 1) / threads);
  launch_chained(swiglu_kernel<elem_t>, dim3(blocks), dim3(threads), 0, (cudaStream_t)stream, (const elem_t*)gate_up, (elem_t*)out,
                                                                     inter, total);
  return check_launch("swiglu");
}

// Rows of a float matrix gathered and cast to T (the rows whose logits are wanted, when the
// stack ends without a norm).
template <typename T>
__global__ void gather_cast_kernel(const float* __restrict__ src, T* __restrict__ dst,
                                   const int* __restrict__ rows, int width) {
  chain_wait();
  const int o = blockIdx.x;
  const float* s = src + (size_t)(rows ? rows[o] : o) * width;
  for (int i = threadIdx.x; i < width; i += blockDim.x) Elem<T>::store(dst + (size_t)o * width + i, s[i]);
}

ERB_EXPORT int erb_gather_cast(const float* src, void* dst, const int* rows, int n_rows, int width,
                               void* stream) {
  if (n_rows <= 0) return ERB_OK;
  launch_chained(gather_cast_kernel<elem_t>, dim3(n_rows), dim3(256), 0, (cudaStream_t)stream, src, (elem_t*)dst, rows, width);
  return check_launch("gather_cast");
}

// ---------------------------------------------------------------------------------------------
// Token ids that are still on the device: an id t < 0 in `ids` stands for row -t - 1 of `fed`, the
// tokens the sampler wrote for the step before (the host launches the next step before it has read
// them).  A row outside `fed` leaves the id negative, which the embedding kernel then flags.
// ---------------------------------------------------------------------------------------------
__global__ void resolve_ids_kernel(int* __restrict__ ids, int n, const int* __restrict__ fed, int n_fed) {
  chain_wait();
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= n) return;
  const int id = ids[t];
  if (id < 0 && -id - 1 < n_fed) ids[t] = fed[-id - 1];
}

ERB_EXPORT int erb_resolve_ids(int* ids, int n, const int* fed, int n_fed, void* stream) {
  if (n <= 0) return ERB_OK;
  if (!ids || !fed || n_fed <= 0) return fail(ERB_ERR_ARG, "resolve_ids: no buffer of fed-back tokens");
  launch_chained(resolve_ids_kernel, dim3((unsigned)((n + 127) / 128)), dim3(128), 0, (cudaStream_t)stream, ids, n, fed, n_fed);
  return check_launch("resolve_ids");
}

// ---------------------------------------------------------------------------------------------
// A gated unit with bounded branches: with g = min(gate, limit) and u = clamp(up, -limit, limit),
//   out[t, i] = g * sigmoid(alpha * g) * (u + shift),      gate = gate_up[t, i], up = gate_up[t, I + i],
// computed in float.  limit <= 0 leaves both branches unbounded; (alpha, shift) = (1, 0) is SwiGLU.  `act` 1 puts
// the tanh form of gelu in the place of g * sigmoid(alpha * g) (see glu_gate).
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void glu_bounded_kernel(const T* __restrict__ gate_up, T* __restrict__ out, int inter, size_t total,
                                   float limit, float alpha, float shift, int act) {
  chain_wait();
  size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const size_t t = idx / inter;
  const int i = (int)(idx % inter);
  const T* row = gate_up + t * 2 * (size_t)inter;
  const float g = Elem<T>::load(row + i), u = Elem<T>::load(row + inter + i);
  Elem<T>::store(out + idx, glu_gate(g, u, act, limit, alpha, shift));
}

// The same on 16-byte groups (the intermediate size a multiple of the group, rows 16-byte aligned).
template <typename T>
__global__ void glu_bounded_vec_kernel(const T* __restrict__ gate_up, T* __restrict__ out, int inter, size_t groups,
                                       float limit, float alpha, float shift, int act) {
  chain_wait();
  constexpr int N = Vec16<T>::N;
  const size_t gidx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (gidx >= groups) return;
  const int per_row = inter / N;
  const size_t t = gidx / per_row;
  const int i = (int)(gidx % per_row) * N;
  const T* row = gate_up + t * 2 * (size_t)inter;
  float g[N], u[N];
  Vec16<T>::load(row + i, g);
  Vec16<T>::load(row + inter + i, u);
#pragma unroll
  for (int j = 0; j < N; ++j) g[j] = glu_gate(g[j], u[j], act, limit, alpha, shift);
  Vec16<T>::store(out + t * (size_t)inter + i, g);
}

ERB_EXPORT int erb_glu_bounded(const void* gate_up, void* out, int n_tokens, int inter, float limit, float alpha,
                               float shift, int act, void* stream) {
  if (n_tokens <= 0) return ERB_OK;
  if (inter <= 0) return fail(ERB_ERR_ARG, "glu_bounded: bad intermediate size");
  const size_t total = (size_t)n_tokens * inter;
  if (inter % Vec16<elem_t>::N == 0 && !((uintptr_t)gate_up & 15) && !((uintptr_t)out & 15)) {
    const size_t groups = total / Vec16<elem_t>::N;
    launch_chained(glu_bounded_vec_kernel<elem_t>, dim3((unsigned)((groups + 255) / 256)), dim3(256), 0, (cudaStream_t)stream,
                   (const elem_t*)gate_up, (elem_t*)out, inter, groups, limit, alpha, shift, act);
    return check_launch("glu_bounded");
  }
  launch_chained(glu_bounded_kernel<elem_t>, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, (cudaStream_t)stream,
                 (const elem_t*)gate_up, (elem_t*)out, inter, total, limit, alpha, shift, act);
  return check_launch("glu_bounded");
}

// ---------------------------------------------------------------------------------------------
// Soft cap of float logits in place: x <- cap * tanh(x / cap), rows `stride` floats apart.
// ---------------------------------------------------------------------------------------------
__global__ void softcap_kernel(float* __restrict__ x, int width, int stride, float cap) {
  chain_wait();
  float* row = x + (size_t)blockIdx.x * stride;
  for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < width; i += gridDim.y * blockDim.x) row[i] = cap * tanhf(row[i] / cap);
}

ERB_EXPORT int erb_softcap(float* x, int n_rows, int width, int stride, float cap, void* stream) {
  if (n_rows <= 0 || width <= 0) return ERB_OK;
  if (!(cap > 0.f) || stride < width) return fail(ERB_ERR_ARG, "softcap: the cap must be positive and the stride cover a row");
  int y = (width + 1023) / 1024;
  if (y > 64) y = 64;
  launch_chained(softcap_kernel, dim3(n_rows, y), dim3(256), 0, (cudaStream_t)stream, x, width, stride, cap);
  return check_launch("softcap");
}

// ---------------------------------------------------------------------------------------------
// Residual add between two layer norms (weight and bias; the variance is the mean of the squared
// deviations from the mean, both taken in float over the whole row):
//   d = delta[row]                       rows of T, or float partial sums added in order and rounded to T
//   d = LN(d; post_w, post_b)            when post_w is given: the norm that closes a sublayer, kept in float
//   r = hidden[row] + d                  stored back when `write_back`
//   out[o] = round_T(LN(r; w, b))        when w is given; round_T(r) when only `out` is; nothing without `out`
// `rows`, when given, selects the rows of hidden/delta that are read; `out` rows are `out_ld` elements apart.
// One block per row; the row is parked in shared memory between the passes.
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256)
add_layernorm_kernel(float* __restrict__ hidden, const T* __restrict__ delta, const float* __restrict__ parts, int n_parts,
                     size_t part_stride, const float* __restrict__ post_w, const float* __restrict__ post_b, float post_eps,
                     const float* __restrict__ w, const float* __restrict__ b, float eps, T* __restrict__ out, int out_ld,
                     const int* __restrict__ rows, int width, int write_back) {
  chain_wait();
  extern __shared__ float row_cache[];  // width floats, then 32 of scratch
  float* scratch = row_cache + width;
  const int o = blockIdx.x;
  const int r = rows ? rows[o] : o;
  float* h = hidden + (size_t)r * width;
  const T* d = delta ? delta + (size_t)r * width : nullptr;
  const float* ps = parts ? parts + (size_t)r * width : nullptr;
  const float inv_w = 1.f / (float)width;
  const bool has_delta = d || ps;
  if (has_delta) {
    float sum = 0.f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
      float v;
      if (d) {
        v = Elem<T>::load(d + i);
      } else {
        v = ps[i];
        for (int sp = 1; sp < n_parts; ++sp) v += ps[sp * part_stride + i];
        v = Elem<T>::round(v);
      }
      row_cache[i] = v;
      sum += v;
    }
    if (post_w) {
      const float mean = block_sum(sum, scratch) * inv_w;
      float sq = 0.f;
      for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const float c = row_cache[i] - mean;
        sq += c * c;
      }
      const float rs = rsqrtf(block_sum(sq, scratch) * inv_w + post_eps);
      for (int i = threadIdx.x; i < width; i += blockDim.x)
        row_cache[i] = (row_cache[i] - mean) * rs * post_w[i] + post_b[i];
    }
  }
  float sum = 0.f;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    float v = h[i];
    if (has_delta) {
      v += row_cache[i];
      if (write_back) h[i] = v;
    }
    row_cache[i] = v;
    sum += v;
  }
  if (!out) return;
  T* y = out + (size_t)o * out_ld;
  if (!w) {
    for (int i = threadIdx.x; i < width; i += blockDim.x) Elem<T>::store(y + i, row_cache[i]);
    return;
  }
  const float mean = block_sum(sum, scratch) * inv_w;
  float sq = 0.f;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    const float c = row_cache[i] - mean;
    sq += c * c;
  }
  const float rs = rsqrtf(block_sum(sq, scratch) * inv_w + eps);
  for (int i = threadIdx.x; i < width; i += blockDim.x)
    Elem<T>::store(y + i, (row_cache[i] - mean) * rs * w[i] + b[i]);
}

// The same with 16-byte accesses and the row in registers: a thread owns up to V groups of four neighbouring
// elements (group g of the row belongs to thread g % blockDim.x), so the row is read once, all of a thread's
// loads are in flight together, and only the four block sums stand between the load and the store.  The sums
// are taken in the order of the kernel above's threads only where the block sizes agree; both kernels are
// within rounding of each other, and a launch always takes the same one for the same width.
template <typename T, int V>
__global__ void __launch_bounds__(256)
add_layernorm_vec4_kernel(float* __restrict__ hidden, const T* __restrict__ delta, const float* __restrict__ parts, int n_parts,
                          size_t part_stride, const float* __restrict__ post_w, const float* __restrict__ post_b, float post_eps,
                          const float* __restrict__ w, const float* __restrict__ b, float eps, T* __restrict__ out, int out_ld,
                          const int* __restrict__ rows, int width, int write_back) {
  __shared__ float scratch[32];
  const int groups = width >> 2;
  const float inv_w = 1.f / (float)width;
  int col[V];
  bool on[V];
#pragma unroll
  for (int v = 0; v < V; ++v) {
    const int g = threadIdx.x + v * blockDim.x;
    on[v] = g < groups;
    col[v] = 4 * g;
  }
  chain_wait();
  const int o = blockIdx.x;
  const int r = rows ? rows[o] : o;
  float* h = hidden + (size_t)r * width;
  const bool has_delta = delta || parts;
  float x[V][4], hv[V][4];
#pragma unroll
  for (int v = 0; v < V; ++v) {
    if (on[v]) load4(h + col[v], hv[v]);
  }
  if (has_delta) {
    float sum = 0.f;
#pragma unroll
    for (int v = 0; v < V; ++v) {
#pragma unroll
      for (int i = 0; i < 4; ++i) x[v][i] = 0.f;
      if (!on[v]) continue;
      if (delta) {
        Pack4<T>::load(delta + (size_t)r * width + col[v], x[v]);
      } else {
        const float* ps = parts + (size_t)r * width + col[v];
        load4(ps, x[v]);
        for (int sp = 1; sp < n_parts; ++sp) {
          float more[4];
          load4(ps + sp * part_stride, more);
#pragma unroll
          for (int i = 0; i < 4; ++i) x[v][i] += more[i];
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) x[v][i] = Elem<T>::round(x[v][i]);
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) sum += x[v][i];
    }
    if (post_w) {
      const float mean = block_sum(sum, scratch) * inv_w;
      float sq = 0.f;
#pragma unroll
      for (int v = 0; v < V; ++v) {
        if (!on[v]) continue;
#pragma unroll
        for (int i = 0; i < 4; ++i) { const float c = x[v][i] - mean; sq += c * c; }
      }
      const float rs = rsqrtf(block_sum(sq, scratch) * inv_w + post_eps);
#pragma unroll
      for (int v = 0; v < V; ++v) {
        if (!on[v]) continue;
        float pw[4], pb[4];
        load4(post_w + col[v], pw);
        load4(post_b + col[v], pb);
#pragma unroll
        for (int i = 0; i < 4; ++i) x[v][i] = (x[v][i] - mean) * rs * pw[i] + pb[i];
      }
    }
  }
  float sum = 0.f;
#pragma unroll
  for (int v = 0; v < V; ++v) {
    if (!on[v]) continue;
    if (has_delta) {
#pragma unroll
      for (int i = 0; i < 4; ++i) hv[v][i] += x[v][i];
      if (write_back) *reinterpret_cast<float4*>(h + col[v]) = make_float4(hv[v][0], hv[v][1], hv[v][2], hv[v][3]);
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) sum += hv[v][i];
  }
  if (!out) return;
  T* y = out + (size_t)o * out_ld;
  if (!w) {
#pragma unroll
    for (int v = 0; v < V; ++v) {
      if (on[v]) Pack4<T>::store(y + col[v], hv[v]);
    }
    return;
  }
  const float mean = block_sum(sum, scratch) * inv_w;
  float sq = 0.f;
#pragma unroll
  for (int v = 0; v < V; ++v) {
    if (!on[v]) continue;
#pragma unroll
    for (int i = 0; i < 4; ++i) { const float c = hv[v][i] - mean; sq += c * c; }
  }
  const float rs = rsqrtf(block_sum(sq, scratch) * inv_w + eps);
#pragma unroll
  for (int v = 0; v < V; ++v) {
    if (!on[v]) continue;
    float ww[4], wb[4], res[4];
    load4(w + col[v], ww);
    load4(b + col[v], wb);
#pragma unroll
    for (int i = 0; i < 4; ++i) res[i] = (hv[v][i] - mean) * rs * ww[i] + wb[i];
    Pack4<T>::store(y + col[v], res);
  }
}

template <int V>
void launch_add_layernorm_vec4(int n_rows, int threads, cudaStream_t stream, float* hidden, const elem_t* delta, const float* parts,
                               int n_parts, size_t part_stride, const float* post_w, const float* post_b, float post_eps,
                               const float* w, const float* b, float eps, elem_t* out, int out_ld, const int* rows, int width,
                               int write_back) {
  launch_chained(add_layernorm_vec4_kernel<elem_t, V>, dim3(n_rows), dim3(threads), 0, stream, hidden, delta, parts, n_parts,
                 part_stride, post_w, post_b, post_eps, w, b, eps, out, out_ld, rows, width, write_back);
}

// delta: rows of the element type, or (n_parts > 0) float partial sums [n_parts][rows of hidden][width].
ERB_EXPORT int erb_add_layernorm(void* hidden, const void* delta, int n_parts, long long part_stride, const float* post_w,
                                 const float* post_b, float post_eps, const float* w, const float* b, float eps, void* out,
                                 int out_ld, const int* rows, int n_rows, int width, int write_back, void* stream) {
  if (n_rows <= 0) return ERB_OK;
  if (width <= 0 || (out && out_ld < width) || (w && !b) || (post_w && !post_b) || (post_w && !delta))
    return fail(ERB_ERR_ARG, "add_layernorm: bad sizes or a weight without its bias");
  const elem_t* d_rows = n_parts > 0 ? (const elem_t*)nullptr : (const elem_t*)delta;
  const float* d_parts = n_parts > 0 ? (const float*)delta : (const float*)nullptr;
  const uintptr_t all = (uintptr_t)hidden | (uintptr_t)delta | (uintptr_t)post_w | (uintptr_t)post_b | (uintptr_t)w | (uintptr_t)b |
                        (uintptr_t)out;
  if (width % 4 == 0 && width <= 8192 && (all & 15) == 0 && out_ld % 8 == 0 && part_stride % 4 == 0) {
    // rows of up to 8,192 elements, everything 16-byte aligned: the row stays in registers
    const int groups = width / 4;
    const int threads = groups >= 256 ? 256 : (groups + 31) / 32 * 32;
    const int per_thread = (groups + threads - 1) / threads;
#define ERB_LN(V) launch_add_layernorm_vec4<V>(n_rows, threads, (cudaStream_t)stream, (float*)hidden, d_rows, d_parts, n_parts,   \
                                               (size_t)part_stride, post_w, post_b, post_eps, w, b, eps, (elem_t*)out, out_ld, rows, \
                                               width, write_back)
    if (per_thread <= 1) ERB_LN(1); else if (per_thread <= 2) ERB_LN(2); else if (per_thread <= 4) ERB_LN(4); else ERB_LN(8);
#undef ERB_LN
    return check_launch("add_layernorm");
  }
  const size_t smem = (size_t)(width + 32) * sizeof(float);
  if (smem > 200 * 1024) return fail(ERB_ERR_UNSUPPORTED, "add_layernorm: width %d does not fit shared memory", width);
  auto kern = add_layernorm_kernel<elem_t>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return fail(ERB_ERR_CUDA, "add_layernorm: %s", cudaGetErrorString(e));
  }
  const int threads = width >= 1024 ? 256 : (width >= 512 ? 128 : 64);
  launch_chained(kern, dim3(n_rows), dim3(threads), smem, (cudaStream_t)stream,
                 (float*)hidden, n_parts > 0 ? (const elem_t*)nullptr : (const elem_t*)delta,
                 n_parts > 0 ? (const float*)delta : (const float*)nullptr, n_parts, (size_t)part_stride, post_w, post_b, post_eps,
                 w, b, eps, (elem_t*)out, out_ld, rows, width, write_back);
  return check_launch("add_layernorm");
}

// ---------------------------------------------------------------------------------------------
// Rows of the float stream cast to T into a wider buffer: dst[t, :width] = round_T(src[t, :]), rows `dst_ld` apart.
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void cast_rows_kernel(const float* __restrict__ src, T* __restrict__ dst, int width, int dst_ld, size_t total) {
  chain_wait();
  const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const size_t t = idx / width;
  const int i = (int)(idx % width);
  Elem<T>::store(dst + t * dst_ld + i, src[idx]);
}

ERB_EXPORT int erb_cast_rows(const float* src, void* dst, int n_rows, int width, int dst_ld, void* stream) {
  if (n_rows <= 0) return ERB_OK;
  if (width <= 0 || dst_ld < width) return fail(ERB_ERR_ARG, "cast_rows: bad sizes");
  const size_t total = (size_t)n_rows * width;
  launch_chained(cast_rows_kernel<elem_t>, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, (cudaStream_t)stream, src,
                 (elem_t*)dst, width, dst_ld, total);
  return check_launch("cast_rows");
}

// ---------------------------------------------------------------------------------------------
// The stream set anew: hidden[t, i] = float(y[t, i]) + vec[i] (a product's rows plus one vector for all rows).
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void stream_set_kernel(float* __restrict__ hidden, const T* __restrict__ y, const float* __restrict__ vec, int width,
                                  size_t total) {
  chain_wait();
  const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  hidden[idx] = Elem<T>::load(y + idx) + (vec ? vec[idx % width] : 0.f);
}

ERB_EXPORT int erb_stream_set(float* hidden, const void* y, const float* vec, int n_rows, int width, void* stream) {
  if (n_rows <= 0) return ERB_OK;
  const size_t total = (size_t)n_rows * width;
  launch_chained(stream_set_kernel<elem_t>, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, (cudaStream_t)stream, hidden,
                 (const elem_t*)y, vec, width, total);
  return check_launch("stream_set");
}

// ---------------------------------------------------------------------------------------------
// Queries and keys made ready for attention, one warp per (token, head) of a row [q heads | k heads | v heads]:
//   x = row[head] (+ bias[head])                                   in float
//   a k head with `values_are_keys`: the token's value row in the cache is round_T(x) (before norm and turn)
//   x = x * rsqrt(mean(x^2) + eps) * norm_w                         when norm weights are given (q_norm for q heads,
//                                                                   k_norm for k heads, one vector for all heads)
//   the first rot_dim entries turned by angle[i] = position * inv_freq[i]: pairs (2i, 2i + 1) when `pairs`, else
//   (i, i + rot_dim / 2); the rest passes
//   q heads are written back in place, k heads to the token's cache slot, v heads (absent with `values_are_keys`)
//   to the slot as they are.  slot = page * page_size + offset, negative: the token writes no key or value.
// ---------------------------------------------------------------------------------------------
constexpr int kPrepWarps = 4;

template <typename T>
__global__ void __launch_bounds__(kPrepWarps * 32)
qk_prepare_kernel(T* __restrict__ qkv, int ld, const float* __restrict__ q_bias, const float* __restrict__ k_bias,
                  const float* __restrict__ q_norm, const float* __restrict__ k_norm, float eps,
                  const int* __restrict__ positions, const float* __restrict__ inv_freq, int rot_dim, int pairs,
                  const int* __restrict__ slots, T* __restrict__ k_pages, T* __restrict__ v_pages, int n_tokens, int nq, int nkv,
                  int D, int page_size, int values_are_keys) {
  chain_wait();
  extern __shared__ float prep_smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float* x = prep_smem + warp * D;
  const int heads = nq + nkv + (values_are_keys ? 0 : nkv);
  const long long item = (long long)blockIdx.x * kPrepWarps + warp;
  if (item >= (long long)n_tokens * heads) return;
  const int t = (int)(item / heads), head = (int)(item % heads);
  T* src = qkv + (size_t)t * ld + (size_t)head * D;
  const int slot = slots ? slots[t] : -1;
  const size_t page = slot >= 0 ? slot / page_size : 0, off = slot >= 0 ? slot % page_size : 0;
  if (head >= nq + nkv) {                        // a value head: copied to the cache as it is
    if (slot < 0 || !v_pages) return;
    T* dst = v_pages + ((page * nkv + (head - nq - nkv)) * page_size + off) * D;
    for (int i = lane; i < D; i += 32) dst[i] = src[i];
    return;
  }
  const bool is_q = head < nq;
  const float* bias = is_q ? q_bias : k_bias;
  if (bias) bias += (size_t)(is_q ? head : head - nq) * D;
  const float* nw = is_q ? q_norm : k_norm;
  const bool store_kv = !is_q && slot >= 0 && k_pages;
  float ss = 0.f;
  for (int i = lane; i < D; i += 32) {
    const float v = Elem<T>::load(src + i) + (bias ? bias[i] : 0.f);
    x[i] = v;
    ss += v * v;
  }
  if (!is_q && values_are_keys && store_kv && v_pages) {
    T* dst = v_pages + ((page * nkv + (head - nq)) * page_size + off) * D;
    for (int i = lane; i < D; i += 32) Elem<T>::store(dst + i, x[i]);
  }
  if (nw) {
    const float rs = rsqrtf(warp_sum(ss) / (float)D + eps);
    for (int i = lane; i < D; i += 32) x[i] = x[i] * rs * nw[i];
  }
  __syncwarp();
  T* dst = is_q ? src : (store_kv ? k_pages + ((page * nkv + (head - nq)) * page_size + off) * D : nullptr);
  if (!dst) return;
  const float pos = (float)positions[t];
  const int half = rot_dim / 2;
  for (int i = lane; i < half; i += 32) {
    const int a = pairs ? 2 * i : i, b = pairs ? 2 * i + 1 : i + half;
    float sn, cs, lo, hi;
    sincosf(pos * inv_freq[i], &sn, &cs);
    rotate_pair(x[a], x[b], cs, sn, lo, hi);
    Elem<T>::store(dst + a, lo);
    Elem<T>::store(dst + b, hi);
  }
  if (!is_q || bias || nw)
    for (int i = rot_dim + lane; i < D; i += 32) Elem<T>::store(dst + i, x[i]);
}

// The same for pairs of neighbours (or no turn at all) and heads of 64, 128 or 256: a lane owns 8 neighbouring
// entries of a head, so a pair never leaves its lane, rows move in 16- or 32-byte pieces, 4, 2 or 1 heads of a
// token are worked on by a warp at a time, and the warp walks `hpw` heads with the token's sines and cosines,
// which it takes once.
template <typename T, int E> struct LaneRow;
template <int E> struct LaneRow<float, E> {
  static __device__ __forceinline__ void load(const float* p, float* v) {
    if constexpr (E == 2) { const float2 r = *reinterpret_cast<const float2*>(p); v[0] = r.x; v[1] = r.y; }
    else {
#pragma unroll
      for (int i = 0; i < E; i += 4) load4(p + i, v + i);
    }
  }
  static __device__ __forceinline__ void store(float* p, const float* v) {
    if constexpr (E == 2) *reinterpret_cast<float2*>(p) = make_float2(v[0], v[1]);
    else {
#pragma unroll
      for (int i = 0; i < E; i += 4) *reinterpret_cast<float4*>(p + i) = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
    }
  }
};
template <int E> struct LaneRow<__nv_bfloat16, E> {
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float* v) {
    uint32_t raw[E / 2];
    if constexpr (E == 2) raw[0] = *reinterpret_cast<const uint32_t*>(p);
    else if constexpr (E == 4) { const uint2 r = *reinterpret_cast<const uint2*>(p); raw[0] = r.x; raw[1] = r.y; }
    else { const uint4 r = *reinterpret_cast<const uint4*>(p); raw[0] = r.x; raw[1] = r.y; raw[2] = r.z; raw[3] = r.w; }
#pragma unroll
    for (int i = 0; i < E / 2; ++i) { v[2 * i] = __uint_as_float(raw[i] << 16); v[2 * i + 1] = __uint_as_float(raw[i] & 0xffff0000u); }
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, const float* v) {
    uint32_t raw[E / 2];
#pragma unroll
    for (int i = 0; i < E / 2; ++i) {
      const __nv_bfloat162 two = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
      raw[i] = *reinterpret_cast<const uint32_t*>(&two);
    }
    if constexpr (E == 2) *reinterpret_cast<uint32_t*>(p) = raw[0];
    else if constexpr (E == 4) *reinterpret_cast<uint2*>(p) = make_uint2(raw[0], raw[1]);
    else *reinterpret_cast<uint4*>(p) = make_uint4(raw[0], raw[1], raw[2], raw[3]);
  }
};

template <typename T, int LPH>   // lanes per head: a lane owns 8 neighbouring entries, so the head size is 8 LPH
__global__ void __launch_bounds__(kPrepWarps * 32)
qk_prepare_lanes_kernel(T* __restrict__ qkv, int ld, const float* __restrict__ q_bias, const float* __restrict__ k_bias,
                        const float* __restrict__ q_norm, const float* __restrict__ k_norm, float eps,
                        const int* __restrict__ positions, const float* __restrict__ inv_freq, int rot_dim,
                        const int* __restrict__ slots, T* __restrict__ k_pages, T* __restrict__ v_pages, int n_tokens, int nq, int nkv,
                        int page_size, int values_are_keys, int hpw) {
  constexpr int E = 8, D = E * LPH, HW = 32 / LPH;       // HW heads of a token are worked on at a time
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, e0 = (lane % LPH) * E, sub = lane / LPH;
  const int heads = nq + nkv + (values_are_keys ? 0 : nkv);
  const int chunks = (heads + hpw - 1) / hpw;
  const int item = blockIdx.x * kPrepWarps + warp;
  // the vectors of the model, read while the kernel before this one drains
  float wq[E], wk[E];
#pragma unroll
  for (int i = 0; i < E; ++i) { wq[i] = q_norm ? q_norm[e0 + i] : 1.f; wk[i] = k_norm ? k_norm[e0 + i] : 1.f; }
  // A head has 4 LPH pairs.  With 8 or 16 lanes per head the warp takes every angle once (lane l those of the pairs
  // l and, with 16, l + 32) and hands them round; with 32 a lane takes the angles of its own four pairs.
  constexpr int OWN = LPH == 32 ? 4 : LPH / 8;            // angles a lane takes
  float freq[OWN];
#pragma unroll
  for (int m = 0; m < OWN; ++m) {
    const int pair = LPH == 32 ? 4 * lane + m : lane + 32 * m;
    freq[m] = 2 * pair < rot_dim ? inv_freq[pair] : 0.f;
  }
  chain_wait();
  if (item >= n_tokens * chunks) return;                  // (a whole warp: the exchanges below are among the lanes that stay)
  const int t = item / chunks, h0 = (item % chunks) * hpw, h1 = min(heads, h0 + hpw);
  // Everything the first round needs from memory is asked for before the angles are taken, so that the loads'
  // latencies overlap each other and the sines and cosines: the position, the slot, the heads' rows and biases.
  const int pos_i = positions[t];
  const int slot = slots ? slots[t] : -1;
  T* row = qkv + (size_t)t * ld + e0;
  float x[E], bb[E];
  bool biased = false;
  auto fetch = [&](int hb) {
    const int head = hb + sub;
#pragma unroll
    for (int i = 0; i < E; ++i) x[i] = 0.f;
    biased = false;
    if (head >= h1) return;
    LaneRow<T, E>::load(row + (size_t)head * D, x);
    const float* bias = head < nq ? q_bias : (head < nq + nkv ? k_bias : nullptr);
    if (bias) {
      LaneRow<float, E>::load(bias + (size_t)(head < nq ? head : head - nq) * D + e0, bb);
      biased = true;
    }
  };
  fetch(h0);
  const float pos = (float)pos_i;
  float own_cs[OWN], own_sn[OWN];
#pragma unroll
  for (int m = 0; m < OWN; ++m) sincosf(pos * freq[m], &own_sn[m], &own_cs[m]);    // (an angle of 0 where nothing is turned)
  float cs[E / 2], sn[E / 2];
#pragma unroll
  for (int j = 0; j < E / 2; ++j) {
    if constexpr (LPH == 32) {
      cs[j] = own_cs[j]; sn[j] = own_sn[j];
    } else {
      const int pair = e0 / 2 + j;                        // this lane's j-th pair; its angle is with lane pair % 32
      float c = __shfl_sync(0xffffffffu, own_cs[0], pair & 31), s = __shfl_sync(0xffffffffu, own_sn[0], pair & 31);
      if constexpr (OWN == 2) {
        const float c1 = __shfl_sync(0xffffffffu, own_cs[1], pair & 31), s1 = __shfl_sync(0xffffffffu, own_sn[1], pair & 31);
        if (pair >= 32) { c = c1; s = s1; }
      }
      cs[j] = c; sn[j] = s;
    }
  }
  const size_t cache_row = slot >= 0 ? ((size_t)(slot / page_size) * nkv * page_size + slot % page_size) * D + e0 : 0;
  const size_t head_step = (size_t)page_size * D;        // from one kv head's row of a page to the next head's
  for (int hb = h0; hb < h1; hb += HW) {
    if (hb > h0) fetch(hb);
    const int head = hb + sub;
    const bool on = head < h1;
    const bool is_v = on && head >= nq + nkv, is_q = on && head < nq, is_k = on && !is_q && !is_v;
    if (biased) {
#pragma unroll
      for (int i = 0; i < E; ++i) x[i] += bb[i];
    }
    if (is_v) {                                  // a value head: copied to the cache as it is
      if (slot >= 0 && v_pages) LaneRow<T, E>::store(v_pages + cache_row + (size_t)(head - nq - nkv) * head_step, x);
    } else if (is_k && values_are_keys && slot >= 0 && k_pages && v_pages) {
      LaneRow<T, E>::store(v_pages + cache_row + (size_t)(head - nq) * head_step, x);
    }
    // the sum of squares over the lanes of a head; every lane of the warp takes part in the exchange
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < E; ++i) ss += x[i] * x[i];
#pragma unroll
    for (int o = LPH / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if (!on || is_v) continue;
    if (is_q ? q_norm != nullptr : k_norm != nullptr) {
      const float rs = rsqrtf(ss / (float)D + eps);
#pragma unroll
      for (int i = 0; i < E; ++i) x[i] = x[i] * rs * (is_q ? wq[i] : wk[i]);
    }
    T* dst = is_q ? row + (size_t)head * D : ((slot >= 0 && k_pages) ? k_pages + cache_row + (size_t)(head - nq) * head_step : nullptr);
    if (!dst) continue;
#pragma unroll
    for (int j = 0; j < E / 2; ++j) {
      if (e0 + 2 * j < rot_dim) {
        float lo, hi;
        rotate_pair(x[2 * j], x[2 * j + 1], cs[j], sn[j], lo, hi);
        x[2 * j] = lo; x[2 * j + 1] = hi;
      }
    }
    LaneRow<T, E>::store(dst, x);
  }
}

template <int LPH>
int launch_qk_prepare_lanes(cudaStream_t stream, elem_t* qkv, int ld, const float* q_bias, const float* k_bias, const float* q_norm,
                            const float* k_norm, float eps, const int* positions, const float* inv_freq, int rot_dim,
                            const int* slots, elem_t* k_pages, elem_t* v_pages, int n_tokens, int nq, int nkv, int page_size,
                            int values_are_keys) {
  constexpr int HW = 32 / LPH;
  const int heads = nq + nkv + (values_are_keys ? 0 : nkv);
  // rounds of HW heads a warp walks: one until there are warps enough to fill the GPU four times over, then up to four
  long long rounds = (long long)n_tokens * heads / (16384LL * HW);
  rounds = rounds < 1 ? 1 : (rounds > 4 ? 4 : rounds);
  const int hpw = (int)rounds * HW;
  const long long items = (long long)n_tokens * ((heads + hpw - 1) / hpw);
  if (items > 0x7fffffffLL) return fail(ERB_ERR_UNSUPPORTED, "qk_prepare: %d tokens of %d heads", n_tokens, heads);
  launch_chained(qk_prepare_lanes_kernel<elem_t, LPH>, dim3((unsigned)((items + kPrepWarps - 1) / kPrepWarps)), dim3(kPrepWarps * 32), 0,
                 stream, qkv, ld, q_bias, k_bias, q_norm, k_norm, eps, positions, inv_freq, rot_dim, slots, k_pages, v_pages, n_tokens,
                 nq, nkv, page_size, values_are_keys, hpw);
  return ERB_OK;
}

ERB_EXPORT int erb_qk_prepare(void* qkv, int ld, const float* q_bias, const float* k_bias, const float* q_norm,
                              const float* k_norm, float eps, const int* positions, const float* inv_freq, int rot_dim,
                              int pairs, const int* slots, void* k_pages, void* v_pages, int n_tokens, int nq, int nkv,
                              int head_dim, int page_size, int values_are_keys, void* stream) {
  if (n_tokens <= 0) return ERB_OK;
  if (nq <= 0 || nkv <= 0 || head_dim <= 0 || rot_dim < 0 || rot_dim > head_dim || rot_dim % 2 || page_size <= 0 || !positions ||
      (rot_dim && !inv_freq))
    return fail(ERB_ERR_ARG, "qk_prepare: bad sizes (rot_dim %d of head_dim %d)", rot_dim, head_dim);
  if (ld < (nq + nkv + (values_are_keys ? 0 : nkv)) * head_dim) return fail(ERB_ERR_ARG, "qk_prepare: rows too narrow");
  const uintptr_t all = (uintptr_t)qkv | (uintptr_t)q_bias | (uintptr_t)k_bias | (uintptr_t)k_pages | (uintptr_t)v_pages;
  if ((pairs || rot_dim == 0) && (head_dim == 64 || head_dim == 128 || head_dim == 256) && ld % 8 == 0 && (all & 15) == 0) {
#define ERB_QK(E) launch_qk_prepare_lanes<E>((cudaStream_t)stream, (elem_t*)qkv, ld, q_bias, k_bias, q_norm, k_norm, eps, positions, \
                                             inv_freq, rot_dim, slots, (elem_t*)k_pages, (elem_t*)v_pages, n_tokens, nq, nkv,        \
                                             page_size, values_are_keys)
    const int rc = head_dim == 64 ? ERB_QK(8) : (head_dim == 128 ? ERB_QK(16) : ERB_QK(32));
#undef ERB_QK
    return rc ? rc : check_launch("qk_prepare");
  }
  const int heads = nq + nkv + (values_are_keys ? 0 : nkv);
  const long long items = (long long)n_tokens * heads;
  const size_t smem = (size_t)kPrepWarps * head_dim * sizeof(float);
  if (smem > 48 * 1024) return fail(ERB_ERR_UNSUPPORTED, "qk_prepare: head_dim %d", head_dim);
  launch_chained(qk_prepare_kernel<elem_t>, dim3((unsigned)((items + kPrepWarps - 1) / kPrepWarps)), dim3(kPrepWarps * 32), smem,
                 (cudaStream_t)stream, (elem_t*)qkv, ld, q_bias, k_bias, q_norm, k_norm, eps, positions, inv_freq, rot_dim, pairs,
                 slots, (elem_t*)k_pages, (elem_t*)v_pages, n_tokens, nq, nkv, head_dim, page_size, values_are_keys);
  return check_launch("qk_prepare");
}

// ---------------------------------------------------------------------------------------------
// The residual add between RMS norms, for blocks whose sublayers read the stream itself and norm what they add:
//   h = hidden[row]                                   float
//   h = h * rsqrt(mean(h^2) + self_eps) * self_w      when self_w is given (the stream normed in place: after the embedding)
//   d = delta[row] (rows of T, or `n_parts` float arrays added in order and rounded to T once) (+ bias, in float)
//   d = d * rsqrt(mean(d^2) + post_eps) * post_w      when post_w is given (the norm that closes the sublayer; stays float)
//   h += d, stored back when `write_back`
//   out[o] = round_T(h)                               when w is null
//          = round_T(h * rsqrt(mean(h^2) + eps) * w)  otherwise
// Every mean, scale and sum is float; eps sits inside the root.  One block per row, the row parked in shared memory.
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256)
rms_between_kernel(float* __restrict__ hidden, const T* __restrict__ delta, const float* __restrict__ parts, int n_parts,
                   size_t part_stride, const float* __restrict__ bias, const float* __restrict__ self_w, float self_eps,
                   const float* __restrict__ post_w, float post_eps, const float* __restrict__ w, float eps,
                   T* __restrict__ out, int out_ld, const int* __restrict__ rows, int width, int write_back) {
  chain_wait();
  extern __shared__ float rb_smem[];     // width floats for the row, width for the update, 32 of scratch
  float* row = rb_smem;
  float* upd = rb_smem + width;
  float* scratch = upd + width;
  const int o = blockIdx.x;
  const int r = rows ? rows[o] : o;
  float* h = hidden + (size_t)r * width;
  const float inv_w = 1.f / (float)width;
  float sq = 0.f;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    const float v = h[i];
    row[i] = v;
    sq += v * v;
  }
  if (self_w) {
    const float rs = rsqrtf(block_sum(sq, scratch) * inv_w + self_eps);
    for (int i = threadIdx.x; i < width; i += blockDim.x) row[i] = row[i] * rs * self_w[i];
  }
  const T* d = delta ? delta + (size_t)r * width : nullptr;
  const float* ps = parts ? parts + (size_t)r * width : nullptr;
  if (d || ps) {
    float dsq = 0.f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
      float v;
      if (d) {
        v = Elem<T>::load(d + i);
      } else {
        v = ps[i];
        for (int sp = 1; sp < n_parts; ++sp) v += ps[sp * part_stride + i];
        v = Elem<T>::round(v);
      }
      if (bias) v += bias[i];
      upd[i] = v;
      dsq += v * v;
    }
    float rs = 1.f;
    if (post_w) rs = rsqrtf(block_sum(dsq, scratch) * inv_w + post_eps);
    for (int i = threadIdx.x; i < width; i += blockDim.x)
      row[i] += post_w ? upd[i] * rs * post_w[i] : upd[i];
  }
  if (write_back && (self_w || d || ps))
    for (int i = threadIdx.x; i < width; i += blockDim.x) h[i] = row[i];
  if (!out) return;
  T* y = out + (size_t)o * out_ld;
  if (!w) {
    for (int i = threadIdx.x; i < width; i += blockDim.x) Elem<T>::store(y + i, row[i]);
    return;
  }
  float s2 = 0.f;
  for (int i = threadIdx.x; i < width; i += blockDim.x) s2 += row[i] * row[i];
  const float rs = rsqrtf(block_sum(s2, scratch) * inv_w + eps);
  for (int i = threadIdx.x; i < width; i += blockDim.x) Elem<T>::store(y + i, row[i] * rs * w[i]);
}

// The same for rows of whole 16-byte pieces without a norm of the stream itself: the row and the update stay in registers
// (V pieces a thread), every load is on its way before the first sum.
template <typename T, int V>
__global__ void __launch_bounds__(256)
rms_between_vec_kernel(float* __restrict__ hidden, const T* __restrict__ delta, const float* __restrict__ parts, int n_parts,
                       size_t part_stride, const float* __restrict__ bias, const float* __restrict__ post_w, float post_eps,
                       const float* __restrict__ w, float eps, T* __restrict__ out, int out_ld, const int* __restrict__ rows,
                       int width, int write_back) {
  chain_wait();
  __shared__ float scratch[32];
  const int o = blockIdx.x;
  const int r = rows ? rows[o] : o;
  float* h = hidden + (size_t)r * width;
  const int n4 = width / 4;
  const float inv_w = 1.f / (float)width;
  float4 row[V], upd[V];
#pragma unroll
  for (int v = 0; v < V; ++v) {
    const int i = threadIdx.x + v * 256;
    row[v] = i < n4 ? reinterpret_cast<const float4*>(h)[i] : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  const bool has_update = delta || parts;
  if (has_update) {
    float dsq = 0.f;
#pragma unroll
    for (int v = 0; v < V; ++v) {
      const int i = threadIdx.x + v * 256;
      float4 u = make_float4(0.f, 0.f, 0.f, 0.f);
      if (i < n4) {
        if (delta) {
          const T* d = delta + (size_t)r * width + 4 * i;
          u = make_float4(Elem<T>::load(d), Elem<T>::load(d + 1), Elem<T>::load(d + 2), Elem<T>::load(d + 3));
        } else {
          const float* ps = parts + (size_t)r * width + 4 * i;
          u = *reinterpret_cast<const float4*>(ps);
          for (int sp = 1; sp < n_parts; ++sp) {
            const float4 q = *reinterpret_cast<const float4*>(ps + sp * part_stride);
            u.x += q.x; u.y += q.y; u.z += q.z; u.w += q.w;
          }
          u = make_float4(Elem<T>::round(u.x), Elem<T>::round(u.y), Elem<T>::round(u.z), Elem<T>::round(u.w));
        }
        if (bias) {
          const float4 b = reinterpret_cast<const float4*>(bias)[i];
          u.x += b.x; u.y += b.y; u.z += b.z; u.w += b.w;
        }
      }
      upd[v] = u;
      dsq += u.x * u.x + u.y * u.y + u.z * u.z + u.w * u.w;
    }
    float rs = 1.f;
    if (post_w) rs = rsqrtf(block_sum(dsq, scratch) * inv_w + post_eps);
#pragma unroll
    for (int v = 0; v < V; ++v) {
      const int i = threadIdx.x + v * 256;
      if (i >= n4) continue;
      float4 pw = make_float4(1.f, 1.f, 1.f, 1.f);
      if (post_w) pw = reinterpret_cast<const float4*>(post_w)[i];
      row[v].x += post_w ? upd[v].x * rs * pw.x : upd[v].x;
      row[v].y += post_w ? upd[v].y * rs * pw.y : upd[v].y;
      row[v].z += post_w ? upd[v].z * rs * pw.z : upd[v].z;
      row[v].w += post_w ? upd[v].w * rs * pw.w : upd[v].w;
      if (write_back) reinterpret_cast<float4*>(h)[i] = row[v];
    }
  }
  if (!out) return;
  T* y = out + (size_t)o * out_ld;
  float rs = 1.f;
  if (w) {
    float s2 = 0.f;
#pragma unroll
    for (int v = 0; v < V; ++v) s2 += row[v].x * row[v].x + row[v].y * row[v].y + row[v].z * row[v].z + row[v].w * row[v].w;
    rs = rsqrtf(block_sum(s2, scratch) * inv_w + eps);
  }
#pragma unroll
  for (int v = 0; v < V; ++v) {
    const int i = threadIdx.x + v * 256;
    if (i >= n4) continue;
    float4 ww = make_float4(1.f, 1.f, 1.f, 1.f);
    if (w) ww = reinterpret_cast<const float4*>(w)[i];
    T* dst = y + 4 * i;
    Elem<T>::store(dst, w ? row[v].x * rs * ww.x : row[v].x);
    Elem<T>::store(dst + 1, w ? row[v].y * rs * ww.y : row[v].y);
    Elem<T>::store(dst + 2, w ? row[v].z * rs * ww.z : row[v].z);
    Elem<T>::store(dst + 3, w ? row[v].w * rs * ww.w : row[v].w);
  }
}

ERB_EXPORT int erb_rms_between(void* hidden, const void* delta, int n_parts, long long part_stride, const float* bias,
                               const float* self_w, float self_eps, const float* post_w, float post_eps, const float* w,
                               float eps, void* out, int out_ld, const int* rows, int n_rows, int width, int write_back,
                               void* stream) {
  if (n_rows <= 0) return ERB_OK;
  if (width <= 0 || (out && out_ld < width)) return fail(ERB_ERR_ARG, "rms_between: bad sizes");
  const size_t smem = sizeof(float) * (2 * (size_t)width + 32);
  if (smem > 200 * 1024) return fail(ERB_ERR_UNSUPPORTED, "rms_between: rows of %d entries", width);
  auto kern = rms_between_kernel<elem_t>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return fail(ERB_ERR_CUDA, "rms_between: %s", cudaGetErrorString(e));
  }
  const bool in_parts = n_parts > 0;
  const bool aligned = !(((uintptr_t)hidden | (uintptr_t)delta | (uintptr_t)bias | (uintptr_t)post_w | (uintptr_t)w) & 15) &&
                       (!in_parts || part_stride % 4 == 0);
  if (!self_w && width % 4 == 0 && width <= 8192 && aligned) {
    const int pieces = (width / 4 + 255) / 256;
#define ERB_RMS_CASE(V)                                                                                                  \
  launch_chained(rms_between_vec_kernel<elem_t, V>, dim3(n_rows), dim3(256), 0, (cudaStream_t)stream, (float*)hidden,     \
                 in_parts ? nullptr : (const elem_t*)delta, in_parts ? (const float*)delta : nullptr, n_parts,          \
                 (size_t)part_stride, bias, post_w, post_eps, w, eps, (elem_t*)out, out_ld, rows, width, write_back)
    if (pieces <= 1) ERB_RMS_CASE(1);
    else if (pieces <= 2) ERB_RMS_CASE(2);
    else if (pieces <= 4) ERB_RMS_CASE(4);
    else ERB_RMS_CASE(8);
#undef ERB_RMS_CASE
    return check_launch("rms_between");
  }
  launch_chained(kern, dim3(n_rows), dim3(width >= 1024 ? 256 : 128), smem, (cudaStream_t)stream, (float*)hidden,
                 in_parts ? nullptr : (const elem_t*)delta, in_parts ? (const float*)delta : nullptr, n_parts,
                 (size_t)part_stride, bias, self_w, self_eps, post_w, post_eps, w, eps, (elem_t*)out, out_ld, rows, width,
                 write_back);
  return check_launch("rms_between");
}

// ---------------------------------------------------------------------------------------------
// Float rows plus one vector: y[t, i] += vec[i] (a bias after a product whose result stayed float).
// ---------------------------------------------------------------------------------------------
__global__ void bias_rows_kernel(float* __restrict__ y, const float* __restrict__ vec, int width, size_t total) {
  chain_wait();
  const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx < total) y[idx] += vec[idx % width];
}

ERB_EXPORT int erb_bias_rows(float* y, const float* vec, int n_rows, int width, void* stream) {
  if (n_rows <= 0) return ERB_OK;
  const size_t total = (size_t)n_rows * width;
  launch_chained(bias_rows_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, (cudaStream_t)stream, y, vec, width, total);
  return check_launch("bias_rows");
}

// ---------------------------------------------------------------------------------------------
// Queries, keys and values of a token made ready for attention where the norm of queries and keys runs over the whole
// projection (all heads of the token at once).  A row is [q: nq heads | k: nkv heads | v: nkv heads], every head D
// entries wide; D may be wider than the true head sizes (the entries beyond them hold zeros and their biases and norm
// weights are zero), so the means divide by the true counts `q_count` and `k_count`.
//   q = row_q + q_bias;  q = q * rsqrt(sum(q^2) / q_count + eps) * q_norm[all entries]      float
//   k likewise with k_bias, k_count, k_norm;   v = row_v + v_bias
//   the first rot_dim entries of every q and k head are turned, entry i with entry i + rot_dim / 2, by position * inv_freq[i]
//   q goes back in place, k and v to the token's cache slot (page * page_size + offset; negative or no pages: not written).
// `has_kv` 0: the row holds queries only (a layer that reads another layer's keys and values).
// One block per token.
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256)
qkv_whole_norm_kernel(T* __restrict__ qkv, int ld, const float* __restrict__ q_bias, const float* __restrict__ k_bias,
                      const float* __restrict__ v_bias, const float* __restrict__ q_norm, const float* __restrict__ k_norm,
                      float q_count, float k_count, float eps, const int* __restrict__ positions,
                      const float* __restrict__ inv_freq, int rot_dim, const int* __restrict__ slots, T* __restrict__ k_pages,
                      T* __restrict__ v_pages, int nq, int nkv, int D, int page_size, int has_kv) {
  chain_wait();
  extern __shared__ float wn_smem[];      // (nq + nkv) * D floats, then 32 of scratch
  const int qw = nq * D, kw = has_kv ? nkv * D : 0;
  float* q_s = wn_smem;
  float* k_s = wn_smem + qw;
  float* scratch = k_s + kw;
  const int t = blockIdx.x;
  T* row = qkv + (size_t)t * ld;
  float sq = 0.f, sk = 0.f;
  for (int i = threadIdx.x; i < qw; i += blockDim.x) {
    const float v = Elem<T>::load(row + i) + (q_bias ? q_bias[i] : 0.f);
    q_s[i] = v;
    sq += v * v;
  }
  for (int i = threadIdx.x; i < kw; i += blockDim.x) {
    const float v = Elem<T>::load(row + qw + i) + (k_bias ? k_bias[i] : 0.f);
    k_s[i] = v;
    sk += v * v;
  }
  const float rq = q_norm ? rsqrtf(block_sum(sq, scratch) / q_count + eps) : 1.f;
  const float rk = (has_kv && k_norm) ? rsqrtf(block_sum(sk, scratch) / k_count + eps) : 1.f;
  __syncthreads();
  const int pos = positions[t];
  const int half = rot_dim / 2;
  const int slot = (has_kv && slots && k_pages) ? slots[t] : -1;
  const int page = slot >= 0 ? slot / page_size : 0, offset = slot >= 0 ? slot % page_size : 0;
  // every thread owns entries (head, i) with i < D - half: i < half is a turned pair (i, i + half), the others pass
  const int per_head = D - half;
  for (int idx = threadIdx.x; idx < (nq + (has_kv ? nkv : 0)) * per_head; idx += blockDim.x) {
    const int head = idx / per_head, j = idx % per_head;
    const bool is_q = head < nq;
    const int hh = is_q ? head : head - nq;
    const float* src = is_q ? q_s + hh * D : k_s + hh * D;
    const float* nw = is_q ? (q_norm ? q_norm + hh * D : nullptr) : (k_norm ? k_norm + hh * D : nullptr);
    const float rs = is_q ? rq : rk;
    T* dst = is_q ? row + hh * D
                  : (slot >= 0 ? k_pages + (((size_t)page * nkv + hh) * page_size + offset) * D : nullptr);
    if (!dst) continue;
    if (j < half) {
      const float a = src[j] * rs * (nw ? nw[j] : 1.f), b = src[j + half] * rs * (nw ? nw[j + half] : 1.f);
      float sn, cs;
      sincosf((float)pos * inv_freq[j], &sn, &cs);
      float lo, hi;
      rotate_pair(a, b, cs, sn, lo, hi);
      Elem<T>::store(dst + j, lo);
      Elem<T>::store(dst + j + half, hi);
    } else {
      const int i = j + half;
      Elem<T>::store(dst + i, src[i] * rs * (nw ? nw[i] : 1.f));
    }
  }
  if (slot >= 0 && v_pages) {
    for (int i = threadIdx.x; i < kw; i += blockDim.x) {
      const int hh = i / D, e = i % D;
      const float v = Elem<T>::load(row + qw + kw + i) + (v_bias ? v_bias[i] : 0.f);
      Elem<T>::store(v_pages + (((size_t)page * nkv + hh) * page_size + offset) * D + e, v);
    }
  }
}

ERB_EXPORT int erb_qkv_whole_norm(void* qkv, int ld, const float* q_bias, const float* k_bias, const float* v_bias,
                                  const float* q_norm, const float* k_norm, int q_count, int k_count, float eps,
                                  const int* positions, const float* inv_freq, int rot_dim, const int* slots, void* k_pages,
                                  void* v_pages, int n_tokens, int nq, int nkv, int head_dim, int page_size, int has_kv,
                                  void* stream) {
  if (n_tokens <= 0) return ERB_OK;
  if (nq <= 0 || nkv <= 0 || head_dim <= 0 || rot_dim < 0 || rot_dim % 2 || rot_dim > head_dim || (rot_dim && !inv_freq) ||
      q_count <= 0 || k_count <= 0 || page_size <= 0)
    return fail(ERB_ERR_ARG, "qkv_whole_norm: bad sizes (rot_dim %d of head_dim %d)", rot_dim, head_dim);
  if (ld < (nq + (has_kv ? 2 * nkv : 0)) * head_dim) return fail(ERB_ERR_ARG, "qkv_whole_norm: rows too narrow");
  const size_t smem = sizeof(float) * ((size_t)(nq + (has_kv ? nkv : 0)) * head_dim + 32);
  if (smem > 200 * 1024) return fail(ERB_ERR_UNSUPPORTED, "qkv_whole_norm: %d heads of %d", nq + nkv, head_dim);
  auto kern = qkv_whole_norm_kernel<elem_t>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return fail(ERB_ERR_CUDA, "qkv_whole_norm: %s", cudaGetErrorString(e));
  }
  launch_chained(kern, dim3(n_tokens), dim3(256), smem, (cudaStream_t)stream, (elem_t*)qkv, ld, q_bias, k_bias, v_bias, q_norm,
                 k_norm, (float)q_count, (float)k_count, eps, positions, inv_freq, rot_dim, slots, (elem_t*)k_pages,
                 (elem_t*)v_pages, nq, nkv, head_dim, page_size, has_kv);
  return check_launch("qkv_whole_norm");
}

// ---------------------------------------------------------------------------------------------
// The activation of a feed-forward without a gate branch: out[t][i] = f(in[t][i]) for i < width, in float, rounded once.
//   act 0: the exact gelu, 0.5 z (1 + erf(z / sqrt 2));  act 1: the square of relu.
// `gate_col` >= 0: column `gate_col` of the input row holds one logit per token, and the row is multiplied by its sigmoid
// (a branch that is scaled as a whole: the scale commutes with the product that follows).
// ---------------------------------------------------------------------------------------------
#define ERB_ACT_GELU_ERF 0
#define ERB_ACT_RELU_SQUARED 1
__device__ __forceinline__ float act_value(float z, int act) {
  if (act == ERB_ACT_RELU_SQUARED) {
    const float r = fmaxf(z, 0.f);
    return r * r;
  }
  return 0.5f * z * (1.f + erff(z * 0.70710678118654752f));
}

template <typename T>
__global__ void act_rows_kernel(const T* __restrict__ in, int ld_in, T* __restrict__ out, int width, int act, int gate_col) {
  chain_wait();
  const T* row = in + (size_t)blockIdx.x * ld_in;
  const float g = gate_col >= 0 ? 1.f / (1.f + expf(-Elem<T>::load(row + gate_col))) : 1.f;
  T* dst = out + (size_t)blockIdx.x * width;
  for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < width; i += gridDim.y * blockDim.x)
    Elem<T>::store(dst + i, act_value(Elem<T>::load(row + i), act) * g);
}

ERB_EXPORT int erb_act_rows(const void* in, int ld_in, void* out, int n_rows, int width, int act, int gate_col, void* stream) {
  if (n_rows <= 0 || width <= 0) return ERB_OK;
  if (ld_in < width || gate_col >= ld_in || (act != ERB_ACT_GELU_ERF && act != ERB_ACT_RELU_SQUARED))
    return fail(ERB_ERR_ARG, "act_rows: bad sizes or activation %d", act);
  int y = (width + 1023) / 1024;
  if (y > 64) y = 64;
  launch_chained(act_rows_kernel<elem_t>, dim3(n_rows, y), dim3(256), 0, (cudaStream_t)stream, (const elem_t*)in, ld_in,
                 (elem_t*)out, width, act, gate_col);
  return check_launch("act_rows");
}

// Float rows times a constant, in place (logits of a head whose model scales them); rows `stride` floats apart.
__global__ void scale_rows_kernel(float* __restrict__ x, int width, int stride, float scale) {
  chain_wait();
  float* row = x + (size_t)blockIdx.x * stride;
  for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < width; i += gridDim.y * blockDim.x) row[i] *= scale;
}

ERB_EXPORT int erb_scale_rows(float* x, int n_rows, int width, int stride, float scale, void* stream) {
  if (n_rows <= 0 || width <= 0) return ERB_OK;
  if (stride < width) return fail(ERB_ERR_ARG, "scale_rows: the stride must cover a row");
  int y = (width + 1023) / 1024;
  if (y > 64) y = 64;
  launch_chained(scale_rows_kernel, dim3(n_rows, y), dim3(256), 0, (cudaStream_t)stream, x, width, stride, scale);
  return check_launch("scale_rows");
}
