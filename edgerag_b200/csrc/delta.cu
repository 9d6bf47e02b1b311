// The gated delta rule over ragged batches, with every request's state kept in a slot between steps.
//
// Per token and head h (queries and keys of head h / (H / G); d entries each, values dv entries):
//   q, k: unit vectors, x / sqrt(sum(x^2) + 1e-6), q also times d^-1/2         (from the convolved, activated rows)
//   beta = sigmoid(b_h),   g = exp(-exp(A_log_h) * softplus(a_h + dt_bias_h))    (b, a: columns of the input product)
//   S <- g S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q               S: d x dv, float, one per request and head
// so the read-out sees the token's own write.  Column p of S depends on the other columns through nothing but k, q, g
// and beta, which gives the kernel its shape: a thread owns up to 16 entries of one column, the threads of a column are
// neighbouring lanes, and per token the two dot products S^T k and S^T q are finished with lane shuffles:
//   a = (S_old^T k)_p,  c = (S_old^T q)_p,   u = beta (v_p - g a),   S_new = g S_old + k u,   o_p = g c + u (k . q).
// Everything here is float whatever the element type T of the rows.  The state is stored transposed, [dv][d], so
// that the lanes of a column read neighbouring addresses.
//
// A request's tokens of one step are neighbours in the batch (rows seq_starts[s] .. seq_starts[s+1]), its slot is
// state_slots[s]; every (request, head, column) is walked by exactly one thread group, token after token, so the
// arithmetic of a token does not depend on how the sequence was cut into steps.
#include "common.cuh"

using namespace erb;

ERB_DEFINE_LAST_ERROR(erb_last_error)

namespace {

__device__ __forceinline__ float silu_f(float v) { return v / (1.f + expf(-v)); }
__device__ __forceinline__ float softplus_f(float v) { return v > 20.f ? v : log1pf(expf(v)); }

constexpr int kDeltaChunk = 16;    // tokens staged in shared memory at a time
constexpr int kDeltaRows = 16;     // entries of a column that a thread holds at most

// grid (H, requests, column blocks); block L * PB threads: thread (l, p) holds rows l, l + L, l + 2L, ... of column p.
template <typename T>
__global__ void __launch_bounds__(512)
delta_scan_kernel(const T* __restrict__ qkv, int channels, const T* __restrict__ proj, int ld, int off_b, int off_a,
                  const float* __restrict__ dt_bias, const float* __restrict__ a_log, float* __restrict__ state,
                  const int* __restrict__ seq_starts, const int* __restrict__ state_slots, float* __restrict__ out,
                  int H, int G, int d, int dv, int L, int PB, float q_scale) {
  chain_wait();
  extern __shared__ float smem[];
  float* k_s = smem;                                   // [chunk][d]
  float* q_s = k_s + kDeltaChunk * d;                  // [chunk][d]
  float* v_s = q_s + kDeltaChunk * d;                  // [chunk][PB]
  float* g_s = v_s + kDeltaChunk * PB;                 // [chunk]
  float* beta_s = g_s + kDeltaChunk;                   // [chunk]
  float* kq_s = beta_s + kDeltaChunk;                  // [chunk]
  const int h = blockIdx.x, seq = blockIdx.y, p0 = blockIdx.z * PB;
  const int kh = h / (H / G);
  const int l = threadIdx.x % L, p = threadIdx.x / L;
  const int col = p0 + p;
  const bool live = col < dv;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
  const int start = seq_starts[seq], n_tok = seq_starts[seq + 1] - start;
  float* s_glob = state + (((size_t)state_slots[seq] * H + h) * dv + (live ? col : 0)) * d;
  float S[kDeltaRows];
#pragma unroll
  for (int i = 0; i < kDeltaRows; ++i) {
    const int n = l + L * i;
    S[i] = (live && n < d) ? s_glob[n] : 0.f;
  }
  const float neg_a = -expf(a_log[h]), bias = dt_bias[h];
  const int off_q = kh * d, off_k = G * d + kh * d, off_v = 2 * G * d + h * dv;
  for (int c0 = 0; c0 < n_tok; c0 += kDeltaChunk) {
    const int nc = min(kDeltaChunk, n_tok - c0);
    __syncthreads();                                   // (the chunk before has been read)
    for (int c = warp; c < nc; c += nwarp) {           // a warp makes a token's unit vectors
      const T* row = qkv + (size_t)(start + c0 + c) * channels;
      float sk = 0.f, sq = 0.f;
      for (int n = lane; n < d; n += 32) {
        const float kv = Elem<T>::load(row + off_k + n), qv = Elem<T>::load(row + off_q + n);
        k_s[c * d + n] = kv;
        q_s[c * d + n] = qv;
        sk = fmaf(kv, kv, sk);
        sq = fmaf(qv, qv, sq);
      }
      const float rk = rsqrtf(warp_sum(sk) + 1e-6f), rq = rsqrtf(warp_sum(sq) + 1e-6f) * q_scale;
      float kq = 0.f;
      for (int n = lane; n < d; n += 32) {
        const float kv = k_s[c * d + n] * rk, qv = q_s[c * d + n] * rq;
        k_s[c * d + n] = kv;
        q_s[c * d + n] = qv;
        kq = fmaf(kv, qv, kq);
      }
      kq = warp_sum(kq);
      if (lane == 0) {
        const T* raw = proj + (size_t)(start + c0 + c) * ld;
        kq_s[c] = kq;
        beta_s[c] = 1.f / (1.f + expf(-Elem<T>::load(raw + off_b + h)));
        g_s[c] = expf(neg_a * softplus_f(Elem<T>::load(raw + off_a + h) + bias));
      }
    }
    for (int idx = threadIdx.x; idx < nc * PB; idx += blockDim.x) {
      const int c = idx / PB, pp = idx % PB;
      v_s[idx] = p0 + pp < dv ? Elem<T>::load(qkv + (size_t)(start + c0 + c) * channels + off_v + p0 + pp) : 0.f;
    }
    __syncthreads();
    for (int c = 0; c < nc; ++c) {
      const float* kc = k_s + c * d;
      const float* qc = q_s + c * d;
      float a = 0.f, b = 0.f;
#pragma unroll
      for (int i = 0; i < kDeltaRows; ++i) {
        const int n = l + L * i;
        if (n < d) {
          a = fmaf(S[i], kc[n], a);
          b = fmaf(S[i], qc[n], b);
        }
      }
      for (int o = 1; o < L; o <<= 1) {                // the lanes of a column: a butterfly, the same sum on each
        a += __shfl_xor_sync(0xffffffffu, a, o);
        b += __shfl_xor_sync(0xffffffffu, b, o);
      }
      const float g = g_s[c];
      const float u = beta_s[c] * (v_s[c * PB + p] - g * a);
#pragma unroll
      for (int i = 0; i < kDeltaRows; ++i) {
        const int n = l + L * i;
        if (n < d) S[i] = fmaf(g, S[i], kc[n] * u);
      }
      if (l == 0 && live) out[(size_t)(start + c0 + c) * H * dv + h * dv + col] = fmaf(g, b, u * kq_s[c]);
    }
  }
  if (live) {
#pragma unroll
    for (int i = 0; i < kDeltaRows; ++i) {
      const int n = l + L * i;
      if (n < d) s_glob[n] = S[i];
    }
  }
}

// One warp per (token, head): out = o / sqrt(mean(o^2) + eps) * weight[entry of the head] * silu(gate), o float.
constexpr int kNormWarps = 4;
template <typename T>
__global__ void __launch_bounds__(kNormWarps * 32)
head_norm_gate_kernel(const float* __restrict__ o, const T* __restrict__ gate, int gate_ld, const float* __restrict__ weight,
                      T* __restrict__ out, int n_items, int H, int dv, float eps) {
  chain_wait();
  const int item = blockIdx.x * kNormWarps + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (item >= n_items) return;
  const int t = item / H, h = item % H;
  const float* src = o + ((size_t)t * H + h) * dv;
  float ss = 0.f;
  for (int i = lane; i < dv; i += 32) ss = fmaf(src[i], src[i], ss);
  const float rs = rsqrtf(warp_sum(ss) / (float)dv + eps);
  const T* gt = gate + (size_t)t * gate_ld + h * dv;
  T* dst = out + ((size_t)t * H + h) * dv;
  for (int i = lane; i < dv; i += 32)
    Elem<T>::store(dst + i, src[i] * rs * weight[i] * silu_f(Elem<T>::load(gt + i)));
}

}  // namespace

ERB_EXPORT int erb_delta_scan(const void* qkv, int channels, const void* proj, int ld, int off_b, int off_a,
                              const float* dt_bias, const float* a_log, float* state, const int* seq_starts,
                              const int* state_slots, float* out, int n_seqs, int n_tokens, int H, int G, int d, int dv,
                              void* stream) {
  if (n_seqs <= 0) return ERB_OK;
  if (H <= 0 || G <= 0 || H % G || d <= 0 || dv <= 0 || d > 32 * kDeltaRows)
    return fail(ERB_ERR_ARG, "delta_scan: bad sizes (%d heads over %d, keys of %d up to %d)", H, G, d, 32 * kDeltaRows);
  if (channels < 2 * G * d + H * dv) return fail(ERB_ERR_ARG, "delta_scan: rows too narrow");
  int L = 1;
  while (L * kDeltaRows < d) L <<= 1;
  // columns per block: whole warps, up to 256 threads, fewer where that gives the GPU too few blocks
  int PB = 256 / L;
  while (PB * L > 32 && PB / 2 >= dv) PB >>= 1;
  while (PB * L > 64 && (long long)H * n_seqs * ((dv + PB - 1) / PB) < 2LL * sm_count()) PB >>= 1;
  const int cblocks = (dv + PB - 1) / PB;
  const size_t smem = sizeof(float) * ((size_t)kDeltaChunk * (2 * d + PB + 3));
  auto kern = delta_scan_kernel<elem_t>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return fail(ERB_ERR_CUDA, "delta_scan: %s", cudaGetErrorString(e));
  }
  launch_chained(kern, dim3(H, n_seqs, cblocks), dim3(L * PB), smem, (cudaStream_t)stream, (const elem_t*)qkv, channels,
                 (const elem_t*)proj, ld, off_b, off_a, dt_bias, a_log, state, seq_starts, state_slots, out, H, G, d, dv, L, PB,
                 1.f / sqrtf((float)d));
  return check_launch("delta_scan");
}

ERB_EXPORT int erb_head_norm_gate(const float* o, const void* gate, int gate_ld, const float* weight, void* out, int n_tokens,
                                  int H, int dv, float eps, void* stream) {
  if (n_tokens <= 0) return ERB_OK;
  if (H <= 0 || dv <= 0) return fail(ERB_ERR_ARG, "head_norm_gate: bad sizes");
  const long long items = (long long)n_tokens * H;
  if (items > 0x7fffffffLL) return fail(ERB_ERR_UNSUPPORTED, "head_norm_gate: %d tokens of %d heads", n_tokens, H);
  launch_chained(head_norm_gate_kernel<elem_t>, dim3((unsigned)((items + kNormWarps - 1) / kNormWarps)), dim3(kNormWarps * 32), 0,
                 (cudaStream_t)stream, o, (const elem_t*)gate, gate_ld, weight, (elem_t*)out, (int)items, H, dv, eps);
  return check_launch("head_norm_gate");
}
