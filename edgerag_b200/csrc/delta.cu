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
// that the lanes of a column read neighbouring addresses.  (The walk issues about 100 instructions a token and warp; a
// first form that indexed its rows with a run-time stride issued 430 and took four times as long.)
//
// Two kernels.  `prepare` is parallel over the tokens and leaves, as floats in a scratch, what the walk needs of a token:
// per key head the unit query (scaled) and the unit key, per head (beta, g, k . q), and the value.  `scan` walks a
// request's tokens; a block stages 16 tokens at a time in shared memory with asynchronous copies, the next 16 on their
// way while these are walked.
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

__device__ __forceinline__ void copy16_async(void* smem_dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(smem_dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void copies_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void copies_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

constexpr int kDeltaChunk = 16;    // tokens staged in shared memory at a time
constexpr int kDeltaRows = 16;     // entries of a column that a thread holds at most
constexpr int kPrepWarps = 4;

__host__ __device__ __forceinline__ int pad4(int v) { return (v + 3) & ~3; }

// The scratch of one step: qk [tokens][G][2][pad4(d)], then sc [tokens][H][4] = (beta, g, k . q, 0), then
// vf [tokens][H][pad4(dv)], all float.
struct DeltaScratch {
  float* qk;
  float* sc;
  float* vf;
};
__host__ __device__ inline size_t delta_scratch_floats(int n_tokens, int H, int G, int d, int dv) {
  return (size_t)n_tokens * ((size_t)G * 2 * pad4(d) + (size_t)H * 4 + (size_t)H * pad4(dv));
}
__host__ __device__ inline DeltaScratch delta_scratch(float* base, int n_tokens, int H, int G, int d, int dv) {
  DeltaScratch s;
  s.qk = base;
  s.sc = s.qk + (size_t)n_tokens * G * 2 * pad4(d);
  s.vf = s.sc + (size_t)n_tokens * H * 4;
  return s;
}

// One warp per (token, key head): the unit vectors, then the scalars and values of the heads that use this key head.
template <typename T>
__global__ void __launch_bounds__(kPrepWarps * 32)
delta_prepare_kernel(const T* __restrict__ qkv, int channels, const T* __restrict__ proj, int ld, int off_b, int off_a,
                     const float* __restrict__ dt_bias, const float* __restrict__ a_log, DeltaScratch out, int n_items, int H,
                     int G, int d, int dv, float q_scale) {
  chain_wait();
  const int item = blockIdx.x * kPrepWarps + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (item >= n_items) return;
  const int t = item / G, kh = item % G;
  const int dp = pad4(d), dvp = pad4(dv), rep = H / G;
  const T* row = qkv + (size_t)t * channels;
  const T* qs = row + kh * d;
  const T* ks = row + G * d + kh * d;
  float sk = 0.f, sq = 0.f;
  for (int n = lane; n < d; n += 32) {
    const float kv = Elem<T>::load(ks + n), qv = Elem<T>::load(qs + n);
    sk = fmaf(kv, kv, sk);
    sq = fmaf(qv, qv, sq);
  }
  // (the roots, the decay and the write strength once per token in double, rounded once: their errors would otherwise
  //  compound along the recurrence)
  const float rk = (float)(1.0 / sqrt((double)warp_sum(sk) + 1e-6));
  const float rq = (float)((double)q_scale / sqrt((double)warp_sum(sq) + 1e-6));
  float* qd = out.qk + ((size_t)t * G + kh) * 2 * dp;
  float* kd = qd + dp;
  float kq = 0.f;
  for (int n = lane; n < dp; n += 32) {
    const float kv = n < d ? Elem<T>::load(ks + n) * rk : 0.f, qv = n < d ? Elem<T>::load(qs + n) * rq : 0.f;
    kd[n] = kv;
    qd[n] = qv;
    kq = fmaf(kv, qv, kq);
  }
  kq = warp_sum(kq);
  const T* raw = proj + (size_t)t * ld;
  for (int r = 0; r < rep; ++r) {
    const int h = kh * rep + r;
    if (lane == 0) {
      const float beta = (float)(1.0 / (1.0 + exp(-(double)Elem<T>::load(raw + off_b + h))));
      const double z = (double)(Elem<T>::load(raw + off_a + h) + dt_bias[h]);
      const float g = (float)exp(-exp((double)a_log[h]) * (z > 30.0 ? z : log1p(exp(z))));
      *reinterpret_cast<float4*>(out.sc + ((size_t)t * H + h) * 4) = make_float4(beta, g, kq, 0.f);
    }
    const T* vs = row + 2 * G * d + h * dv;
    float* vd = out.vf + ((size_t)t * H + h) * dvp;
    for (int n = lane; n < dvp; n += 32) vd[n] = n < dv ? Elem<T>::load(vs + n) : 0.f;
  }
}

// grid (H, requests, column blocks); block L * PB threads: thread (l, p) holds 16 rows of column p, four runs of four
// neighbours: rows 4 (l + L j) .. + 3 for j = 0 .. 3, so that the lanes of a column read neighbouring 16-byte pieces of a
// key.  PB is a multiple of 4.  Shared memory: two stages of [chunk][2][16 L] + [chunk][PB] + [chunk][4] floats; a staged
// query or key has room for 16 L entries, the ones past pad4(d) zeroed once, so that the walk reads without a test.
template <int L>
__global__ void __launch_bounds__(512)
delta_scan_kernel(DeltaScratch in, float* __restrict__ state, const int* __restrict__ seq_starts,
                  const int* __restrict__ state_slots, float* __restrict__ out, int H, int G, int d, int dv, int PB) {
  chain_wait();
  extern __shared__ __align__(16) float smem[];
  const int dp = pad4(d), dvp = pad4(dv);
  constexpr int RS = 16 * L;                                   // floats of a staged query or key
  const int stage_floats = kDeltaChunk * (2 * RS + PB + 4);
  const int h = blockIdx.x, seq = blockIdx.y, p0 = blockIdx.z * PB;
  const int kh = h / (H / G);
  const int l = threadIdx.x % L, p = threadIdx.x / L;
  const int col = p0 + p;
  const bool live = col < dv;
  const int start = seq_starts[seq], n_tok = seq_starts[seq + 1] - start;
  float* s_glob = state + (((size_t)state_slots[seq] * H + h) * dv + (live ? col : 0)) * d;
  int row_of[4];                                               // first row of each run
#pragma unroll
  for (int j = 0; j < 4; ++j) row_of[j] = 4 * (l + L * j);
  if (dp < RS) {                                               // the tails that no copy writes
    for (int idx = threadIdx.x; idx < 2 * kDeltaChunk * 2 * (RS - dp); idx += blockDim.x) {
      const int row = idx / (RS - dp), e = idx % (RS - dp);   // row: (stage, token, q or k)
      smem[(row / (2 * kDeltaChunk)) * stage_floats + (row % (2 * kDeltaChunk)) * RS + dp + e] = 0.f;
    }
  }
  float S[kDeltaRows];
#pragma unroll
  for (int i = 0; i < kDeltaRows; ++i) {
    const int n = row_of[i / 4] + (i & 3);
    S[i] = (live && n < d) ? s_glob[n] : 0.f;
  }
  const int qk4 = 2 * dp / 4, v4 = PB / 4;                     // 16-byte pieces of a token's rows
  const int pb_live = min(PB, dvp - p0);                       // columns of this block that the scratch holds
  auto stage = [&](int c0, int buf) {
    float* qk_s = smem + buf * stage_floats;
    float* v_s = qk_s + kDeltaChunk * 2 * RS;
    float* sc_s = v_s + kDeltaChunk * PB;
    const int nc = min(kDeltaChunk, n_tok - c0);
    for (int idx = threadIdx.x; idx < nc * qk4; idx += blockDim.x) {
      const int c = idx / qk4, j = idx % qk4;                  // piece j of the token's [q | k]: to row 2 c or 2 c + 1
      const int which = 4 * j >= dp, e = 4 * j - which * dp;
      copy16_async(qk_s + (2 * c + which) * RS + e, in.qk + ((size_t)(start + c0 + c) * G + kh) * 2 * dp + 4 * j);
    }
    for (int idx = threadIdx.x; idx < nc * v4; idx += blockDim.x) {
      const int c = idx / v4, j = idx % v4;
      if (4 * j < pb_live) copy16_async(v_s + c * PB + 4 * j, in.vf + ((size_t)(start + c0 + c) * H + h) * dvp + p0 + 4 * j);
    }
    for (int c = threadIdx.x; c < nc; c += blockDim.x)
      copy16_async(sc_s + 4 * c, in.sc + ((size_t)(start + c0 + c) * H + h) * 4);
    copies_commit();
  };
  if (n_tok > 0) stage(0, 0);
  float* out_p = out + (size_t)start * H * dv + h * dv + col;
  for (int c0 = 0, buf = 0; c0 < n_tok; c0 += kDeltaChunk, buf ^= 1) {
    const int nc = min(kDeltaChunk, n_tok - c0);
    if (c0 + kDeltaChunk < n_tok) {
      stage(c0 + kDeltaChunk, buf ^ 1);                        // (that stage was read two rounds ago: the barrier below has passed)
      copies_wait<1>();
    } else {
      copies_wait<0>();
    }
    __syncthreads();
    const float* qk_s = smem + buf * stage_floats;
    const float* v_s = qk_s + kDeltaChunk * 2 * RS;
    const float* sc_s = v_s + kDeltaChunk * PB;
#pragma unroll 2
    for (int c = 0; c < nc; ++c) {
      const float* qc = qk_s + c * 2 * RS;
      const float* kc = qc + RS;
      float4 kv[4], qv[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        kv[j] = *reinterpret_cast<const float4*>(kc + row_of[j]);
        qv[j] = *reinterpret_cast<const float4*>(qc + row_of[j]);
      }
      float a0 = 0.f, a1 = 0.f, b0 = 0.f, b1 = 0.f;
#pragma unroll
      for (int j = 0; j < 4; j += 2) {
        a0 = fmaf(S[4 * j], kv[j].x, a0); a0 = fmaf(S[4 * j + 1], kv[j].y, a0);
        a0 = fmaf(S[4 * j + 2], kv[j].z, a0); a0 = fmaf(S[4 * j + 3], kv[j].w, a0);
        b0 = fmaf(S[4 * j], qv[j].x, b0); b0 = fmaf(S[4 * j + 1], qv[j].y, b0);
        b0 = fmaf(S[4 * j + 2], qv[j].z, b0); b0 = fmaf(S[4 * j + 3], qv[j].w, b0);
        a1 = fmaf(S[4 * j + 4], kv[j + 1].x, a1); a1 = fmaf(S[4 * j + 5], kv[j + 1].y, a1);
        a1 = fmaf(S[4 * j + 6], kv[j + 1].z, a1); a1 = fmaf(S[4 * j + 7], kv[j + 1].w, a1);
        b1 = fmaf(S[4 * j + 4], qv[j + 1].x, b1); b1 = fmaf(S[4 * j + 5], qv[j + 1].y, b1);
        b1 = fmaf(S[4 * j + 6], qv[j + 1].z, b1); b1 = fmaf(S[4 * j + 7], qv[j + 1].w, b1);
      }
      float a = a0 + a1, b = b0 + b1;
#pragma unroll
      for (int o = 1; o < L; o <<= 1) {                // the lanes of a column: a butterfly, the same sum on each
        a += __shfl_xor_sync(0xffffffffu, a, o);
        b += __shfl_xor_sync(0xffffffffu, b, o);
      }
      const float4 sc = *reinterpret_cast<const float4*>(sc_s + 4 * c);     // beta, g, k . q
      const float g = sc.y;
      const float u = sc.x * (v_s[c * PB + p] - g * a);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        S[4 * j] = fmaf(g, S[4 * j], kv[j].x * u);
        S[4 * j + 1] = fmaf(g, S[4 * j + 1], kv[j].y * u);
        S[4 * j + 2] = fmaf(g, S[4 * j + 2], kv[j].z * u);
        S[4 * j + 3] = fmaf(g, S[4 * j + 3], kv[j].w * u);
      }
      if (l == 0 && live) out_p[(size_t)(c0 + c) * H * dv] = fmaf(g, b, u * sc.z);
    }
    __syncthreads();                                   // (the stage is free for the copies of the round after next)
  }
  if (live) {
#pragma unroll
    for (int i = 0; i < kDeltaRows; ++i) {
      const int n = row_of[i / 4] + (i & 3);
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

// Floats of the scratch that erb_delta_scan needs for a step of n_tokens tokens.
ERB_EXPORT long long erb_delta_scratch_floats(int n_tokens, int H, int G, int d, int dv) {
  return (long long)delta_scratch_floats(n_tokens, H, G, d, dv);
}

ERB_EXPORT int erb_delta_scan(const void* qkv, int channels, const void* proj, int ld, int off_b, int off_a,
                              const float* dt_bias, const float* a_log, float* state, const int* seq_starts,
                              const int* state_slots, float* out, float* scratch, int n_seqs, int n_tokens, int H, int G, int d,
                              int dv, void* stream) {
  if (n_seqs <= 0 || n_tokens <= 0) return ERB_OK;
  if (H <= 0 || G <= 0 || H % G || d <= 0 || dv <= 0 || d > 32 * kDeltaRows)
    return fail(ERB_ERR_ARG, "delta_scan: bad sizes (%d heads over %d, keys of %d up to %d)", H, G, d, 32 * kDeltaRows);
  if (channels < 2 * G * d + H * dv) return fail(ERB_ERR_ARG, "delta_scan: rows too narrow");
  if (!scratch || ((uintptr_t)scratch & 15)) return fail(ERB_ERR_ARG, "delta_scan: the scratch must be 16-byte aligned");
  const DeltaScratch sc = delta_scratch(scratch, n_tokens, H, G, d, dv);
  const long long items = (long long)n_tokens * G;
  if (items > 0x7fffffffLL) return fail(ERB_ERR_UNSUPPORTED, "delta_scan: %d tokens of %d key heads", n_tokens, G);
  launch_chained(delta_prepare_kernel<elem_t>, dim3((unsigned)((items + kPrepWarps - 1) / kPrepWarps)), dim3(kPrepWarps * 32), 0,
                 (cudaStream_t)stream, (const elem_t*)qkv, channels, (const elem_t*)proj, ld, off_b, off_a, dt_bias, a_log, sc,
                 (int)items, H, G, d, dv, 1.f / sqrtf((float)d));
  int rc = check_launch("delta_prepare");
  if (rc) return rc;
  int L = 1;
  while (L * kDeltaRows < d) L <<= 1;
  // columns per block: whole warps, up to 256 threads, fewer where that gives the GPU too few blocks; at least 4
  int PB = 256 / L;
  while (PB * L > 32 && PB / 2 >= dv && PB > 4) PB >>= 1;
  while (PB * L > 64 && PB > 4 && (long long)H * n_seqs * ((dv + PB - 1) / PB) < 2LL * sm_count()) PB >>= 1;
  const int cblocks = (dv + PB - 1) / PB;
  const size_t smem = sizeof(float) * 2 * ((size_t)kDeltaChunk * (2 * 16 * L + PB + 4));
#define ERB_DELTA_CASE(LL)                                                                                              \
  case LL: {                                                                                                            \
    auto kern = delta_scan_kernel<LL>;                                                                                  \
    if (smem > 48 * 1024) {                                                                                             \
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);               \
      if (e != cudaSuccess) return fail(ERB_ERR_CUDA, "delta_scan: %s", cudaGetErrorString(e));                        \
    }                                                                                                                   \
    launch_chained(kern, dim3(H, n_seqs, cblocks), dim3(LL * PB), smem, (cudaStream_t)stream, sc, state, seq_starts,    \
                   state_slots, out, H, G, d, dv, PB);                                                                  \
  } break;
  switch (L) {
    ERB_DELTA_CASE(1)
    ERB_DELTA_CASE(2)
    ERB_DELTA_CASE(4)
    ERB_DELTA_CASE(8)
    ERB_DELTA_CASE(16)
    default:
      ERB_DELTA_CASE(32)
  }
#undef ERB_DELTA_CASE
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
