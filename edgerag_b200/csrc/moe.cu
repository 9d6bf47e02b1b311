// A feed-forward of routed experts over a ragged batch, without a host round trip: every launch has a shape that
// depends on the number of tokens only, and the kernels find their work in lists made on the device.
//
//   1. route:   z = W_router x (float), s = sigmoid(z); the `top` experts with the largest z (the lower index wins a tie);
//               per token the chosen experts and their scores s.  A (token, choice) is a "pair", numbered token * top + choice.
//   2. lists:   one block per expert counts all choices, makes its offset (and its offset in row tiles) and writes the
//               pair numbers of its expert in rising order behind the offset.
//   3. gate/up: for every expert the rows of its pairs, each row the token's input times the pair's score (rounded to T
//               once), times [W_gate; W_up]^T; act = silu(gate) * up, stored in the order of the lists.
//   4. down:    act times W_down^T, stored as float at [choice][token][:]: the partial sums of the tokens' updates, which
//               whoever adds the update sums in the order of the choices.
// The products walk k in one fixed order whatever tile a row falls into, so a token's result does not depend on the
// other tokens of the step.  Accumulation is float; T is the type of the operands.
#include "common.cuh"

using namespace erb;

ERB_DEFINE_LAST_ERROR(erb_last_error)

// how a router turns logits into scores
#define ERB_SCORE_SIGMOID 0
#define ERB_SCORE_SOFTMAX 1
// what a product of the experts does: the down product, the gated pair of products, a single product with an activation
#define ERB_MOE_DOWN 0
#define ERB_MOE_GATED 1
#define ERB_MOE_SINGLE 2
#define ERB_ACT_RELU_SQUARED 1

namespace {

constexpr int kRouteThreads = 512;

// One block per kRouteTokens tokens.  Shared memory: their logits, then their rows as floats.  A warp takes an expert at
// a time and reads its router row once for all the block's tokens; a lane sums the entries 4 lane .. 4 lane + 3 of every
// run of 128, then the lanes are added: one order of sums per token whatever the batch.  Then a warp per token picks.
constexpr int kRouteTokens = 4;
template <typename T>
__global__ void __launch_bounds__(kRouteThreads)
moe_route_kernel(const T* __restrict__ x, int ld, const float* __restrict__ w_router, int n_tokens, int width, int n_experts,
                 int top, int* __restrict__ choice, float* __restrict__ score, int score_kind, int n_groups, int keep_groups) {
  chain_wait();
  extern __shared__ float z_s[];                 // [kRouteTokens][n_experts padded to 4] logits, the same again for the
  const int e_pad = (n_experts + 3) & ~3;        // groups' maxima, then [kRouteTokens][width]
  float* g_s = z_s + kRouteTokens * e_pad;
  float* x_s = g_s + kRouteTokens * e_pad;
  const int t0 = blockIdx.x * kRouteTokens, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int n_here = min(kRouteTokens, n_tokens - t0);
#pragma unroll
  for (int j = 0; j < kRouteTokens; ++j) {
    const T* row = x + (size_t)(t0 + min(j, n_here - 1)) * ld;
#pragma unroll 4
    for (int k = threadIdx.x; k < width; k += kRouteThreads) x_s[j * width + k] = Elem<T>::load(row + k);
  }
  __syncthreads();
  const int whole = (width & 3) == 0 ? width & ~127 : 0;       // entries read as float4 by whole warps
  for (int e = warp; e < n_experts; e += kRouteThreads / 32) {
    const float* w = w_router + (size_t)e * width;
    float acc[kRouteTokens];
#pragma unroll
    for (int j = 0; j < kRouteTokens; ++j) acc[j] = 0.f;
#pragma unroll 8
    for (int k = 4 * lane; k < whole; k += 128) {            // (eight 16-byte reads of the router's row in flight a lane)
      const float4 wv = *reinterpret_cast<const float4*>(w + k);
#pragma unroll
      for (int j = 0; j < kRouteTokens; ++j) {
        const float4 xv = *reinterpret_cast<const float4*>(x_s + j * width + k);
        acc[j] = fmaf(xv.x, wv.x, acc[j]);
        acc[j] = fmaf(xv.y, wv.y, acc[j]);
        acc[j] = fmaf(xv.z, wv.z, acc[j]);
        acc[j] = fmaf(xv.w, wv.w, acc[j]);
      }
    }
    for (int k = whole + lane; k < width; k += 32) {
      const float wv = w[k];
#pragma unroll
      for (int j = 0; j < kRouteTokens; ++j) acc[j] = fmaf(x_s[j * width + k], wv, acc[j]);
    }
#pragma unroll
    for (int j = 0; j < kRouteTokens; ++j) {
      const float total = warp_sum(acc[j]);
      if (lane == 0) z_s[j * e_pad + e] = total;
    }
  }
  __syncthreads();
  if (warp >= n_here) return;
  const int t = t0 + warp;
  float* z = z_s + warp * e_pad;
  // softmax scores: the maximum and the denominator over all experts, before any expert is ruled out
  float z_top = 0.f, denom = 1.f;
  if (score_kind == ERB_SCORE_SOFTMAX) {
    float mx = -INFINITY;
    for (int e = lane; e < n_experts; e += 32) mx = fmaxf(mx, z[e]);
    z_top = warp_max(mx);
    float sum = 0.f;
    for (int e = lane; e < n_experts; e += 32) sum += expf(z[e] - z_top);
    denom = warp_sum(sum);
  }
  // groups of neighbouring experts: a group's score is its largest logit (the scores rise with the logits); the experts
  // of all but the `keep_groups` best groups are ruled out (the lower group wins a tie)
  if (n_groups > 1 && keep_groups < n_groups) {
    float* gm = g_s + warp * e_pad;
    const int per = n_experts / n_groups;
    for (int g = lane; g < n_groups; g += 32) {
      float mx = -INFINITY;
      for (int e = g * per; e < (g + 1) * per; ++e) mx = fmaxf(mx, z[e]);
      gm[g] = mx;
    }
    __syncwarp();
    for (int c = 0; c < keep_groups; ++c) {
      float best = -INFINITY;
      int arg = 0x7fffffff;
      for (int g = lane; g < n_groups; g += 32) {
        const float v = gm[g];
        if (v > best) { best = v; arg = g; }     // (a group already kept holds NaN: never greater)
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
        if (ob > best || (ob == best && oa < arg)) { best = ob; arg = oa; }
      }
      if (lane == 0 && arg < n_groups) gm[arg] = __int_as_float(0x7fc00000);
      __syncwarp();
    }
    for (int e = lane; e < n_experts; e += 32)
      if (gm[e / per] == gm[e / per]) z[e] = -INFINITY;       // not NaN: the group was not kept
    __syncwarp();
  }
  for (int c = 0; c < top; ++c) {
    float best = -INFINITY;
    int arg = 0x7fffffff;
    for (int e = lane; e < n_experts; e += 32) {
      const float zv = z[e];
      if (zv > best) { best = zv; arg = e; }     // rising e within a lane: the first maximum stays
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
      if (ob > best || (ob == best && oa < arg)) { best = ob; arg = oa; }
    }
    if (lane == 0) {
      choice[(size_t)t * top + c] = arg;
      score[(size_t)t * top + c] = score_kind == ERB_SCORE_SOFTMAX ? expf(best - z_top) / denom : 1.f / (1.f + expf(-best));
      z[arg] = -INFINITY;
    }
    __syncwarp();
  }
}

// One block per expert e builds the expert's part of the lists on its own: a histogram of all choices in shared memory
// gives offsets[e] (the pairs of the experts before e) and tiles[e] (their row tiles of `tile_rows` rows); then the pairs
// that chose e are written behind the offset in rising order.  The last block also writes the totals at [n_experts].
__global__ void __launch_bounds__(256) moe_lists_kernel(const int* __restrict__ choice, int n_pairs, int n_experts, int tile_rows,
                                                        int* __restrict__ counts, int* __restrict__ offsets,
                                                        int* __restrict__ tiles, int* __restrict__ order) {
  chain_wait();
  extern __shared__ int hist[];                  // [n_experts]
  __shared__ int warp_counts[8];
  __shared__ int base_s;
  const int e = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int i = threadIdx.x; i < n_experts; i += blockDim.x) hist[i] = 0;
  __syncthreads();
  for (int i = threadIdx.x; i < n_pairs; i += blockDim.x) atomicAdd(&hist[choice[i]], 1);
  __syncthreads();
  if (threadIdx.x == 0) {
    int off = 0, tl = 0;
    for (int i = 0; i < e; ++i) {
      off += hist[i];
      tl += (hist[i] + tile_rows - 1) / tile_rows;
    }
    counts[e] = hist[e];
    offsets[e] = off;
    tiles[e] = tl;
    base_s = off;
    if (e == n_experts - 1) {
      offsets[n_experts] = off + hist[e];
      tiles[n_experts] = tl + (hist[e] + tile_rows - 1) / tile_rows;
      counts[n_experts] = 0;
    }
  }
  __syncthreads();
  for (int i0 = 0; i0 < n_pairs; i0 += 256) {
    const int i = i0 + threadIdx.x;
    const bool mine = i < n_pairs && choice[i] == e;
    const unsigned ballot = __ballot_sync(0xffffffffu, mine);
    if (lane == 0) warp_counts[warp] = __popc(ballot);
    __syncthreads();
    int before = 0;
    for (int w = 0; w < warp; ++w) before += warp_counts[w];
    if (mine) order[base_s + before + __popc(ballot & ((1u << lane) - 1))] = i;
    __syncthreads();
    if (threadIdx.x == 0) {
      int all = 0;
      for (int w = 0; w < 8; ++w) all += warp_counts[w];
      base_s += all;
    }
    __syncthreads();
  }
}

// ---------------------------------------------------------------------------------------------
// The experts' products on CUDA cores: a block owns TM rows of one expert's list and TN columns; k is walked in
// steps of BK in rising order with one float accumulator per output.
//   GATED:  rows are gathered inputs (times the pair's score where `score` is given, rounded to T once), the weight holds
//           `n_out` gate rows followed by `n_out` up rows, the output is silu(gate) * up in T at the row's place in the list;
//   SINGLE: the same rows against `n_out` rows of one weight, the output is act(product) in T (act: the square of relu);
//   DOWN:   rows are the list's rows of `a`, the output is float at [choice][token][:], times the pair's score where
//           `score` is given (an expert's output weighted by its score).
// ---------------------------------------------------------------------------------------------
constexpr int kTM = 32, kTN = 64, kBK = 32;

template <typename T, int MODE>
__global__ void __launch_bounds__(256)
moe_product_kernel(const T* __restrict__ a, int lda, const T* __restrict__ weights, const int* __restrict__ offsets,
                   const int* __restrict__ tiles, const int* __restrict__ order, const float* __restrict__ score, int n_experts,
                   int top, int n_tokens, int n_out, int k_dim, T* __restrict__ act, float* __restrict__ parts) {
  chain_wait();
  constexpr bool GATED = MODE == ERB_MOE_GATED, GATHER = MODE != ERB_MOE_DOWN;
  __shared__ float a_s[kTM][kBK + 1];
  __shared__ float b_s[kTN][kBK + 1];
  __shared__ float b2_s[GATED ? kTN : 1][kBK + 1];
  __shared__ int pair_s[kTM];
  __shared__ float scale_s[kTM];
  const int tile = blockIdx.x;
  if (tile >= tiles[n_experts]) return;
  int e = 0;
  {
    int lo = 0, hi = n_experts;                          // the last e with tiles[e] <= tile
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (tiles[mid] <= tile) lo = mid; else hi = mid;
    }
    e = lo;
  }
  const int row0 = offsets[e] + (tile - tiles[e]) * kTM;
  const int n_rows = min(kTM, offsets[e + 1] - row0);
  const int col0 = blockIdx.y * kTN;
  if (threadIdx.x < kTM) {
    const int r = threadIdx.x;
    const int pair = r < n_rows ? order[row0 + r] : -1;
    pair_s[r] = pair;
    scale_s[r] = (score && pair >= 0) ? score[pair] : 1.f;
  }
  __syncthreads();
  const T* w = weights + (size_t)e * (GATED ? 2 : 1) * n_out * k_dim;
  const int ty = threadIdx.x / 16, tx = threadIdx.x % 16;   // rows 2 ty, 2 ty + 1; columns tx + 16 j
  float acc[2][4] = {}, acc2[2][4] = {};
  for (int k0 = 0; k0 < k_dim; k0 += kBK) {
    for (int idx = threadIdx.x; idx < kTM * kBK; idx += 256) {
      const int r = idx / kBK, kk = idx % kBK;
      float v = 0.f;
      if (r < n_rows && k0 + kk < k_dim) {
        if (GATHER) v = Elem<T>::round(scale_s[r] * Elem<T>::load(a + (size_t)(pair_s[r] / top) * lda + k0 + kk));
        else v = Elem<T>::load(a + (size_t)(row0 + r) * lda + k0 + kk);
      }
      a_s[r][kk] = v;
    }
    for (int idx = threadIdx.x; idx < kTN * kBK; idx += 256) {
      const int c = idx / kBK, kk = idx % kBK;
      const bool ok = col0 + c < n_out && k0 + kk < k_dim;
      b_s[c][kk] = ok ? Elem<T>::load(w + (size_t)(col0 + c) * k_dim + k0 + kk) : 0.f;
      if (GATED) b2_s[c][kk] = ok ? Elem<T>::load(w + (size_t)(n_out + col0 + c) * k_dim + k0 + kk) : 0.f;
    }
    __syncthreads();
#pragma unroll 8
    for (int kk = 0; kk < kBK; ++kk) {
      const float a0 = a_s[2 * ty][kk], a1 = a_s[2 * ty + 1][kk];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float b = b_s[tx + 16 * j][kk];
        acc[0][j] = fmaf(a0, b, acc[0][j]);
        acc[1][j] = fmaf(a1, b, acc[1][j]);
        if (GATED) {
          const float b2 = b2_s[tx + 16 * j][kk];
          acc2[0][j] = fmaf(a0, b2, acc2[0][j]);
          acc2[1][j] = fmaf(a1, b2, acc2[1][j]);
        }
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int r = 2 * ty + i;
    if (r >= n_rows) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int c = col0 + tx + 16 * j;
      if (c >= n_out) continue;
      if (GATED) {
        Elem<T>::store(act + (size_t)(row0 + r) * n_out + c, silu_mul(acc[i][j], acc2[i][j]));
      } else if (MODE == ERB_MOE_SINGLE) {
        const float z = fmaxf(acc[i][j], 0.f);
        Elem<T>::store(act + (size_t)(row0 + r) * n_out + c, z * z);
      } else {
        const int pair = pair_s[r];
        parts[((size_t)(pair % top) * n_tokens + pair / top) * n_out + c] = acc[i][j] * scale_s[r];
      }
    }
  }
}

}  // namespace

ERB_EXPORT int erb_moe_tile_rows() { return kTM; }

ERB_EXPORT int erb_moe_route(const void* x, int ld, const float* w_router, int n_tokens, int width, int n_experts, int top,
                             int* choice, float* score, int* counts, int* offsets, int* tiles, int* order, int tile_rows,
                             int score_kind, int n_groups, int keep_groups, void* stream) {
  if (n_tokens <= 0) return ERB_OK;
  if (width <= 0 || n_experts <= 0 || top <= 0 || top > n_experts || n_experts > 8192)
    return fail(ERB_ERR_ARG, "moe_route: %d of %d experts", top, n_experts);
  if ((score_kind != ERB_SCORE_SIGMOID && score_kind != ERB_SCORE_SOFTMAX) || n_groups < 1 || n_experts % n_groups ||
      keep_groups < 1 || keep_groups > n_groups || top > keep_groups * (n_experts / n_groups))
    return fail(ERB_ERR_ARG, "moe_route: %d groups of which %d are kept cannot give %d of %d experts", n_groups, keep_groups, top,
                n_experts);
  cudaStream_t s = (cudaStream_t)stream;
  const int n_pairs = n_tokens * top;
  const size_t route_smem = sizeof(float) * kRouteTokens * (2 * (size_t)((n_experts + 3) & ~3) + width);
  if (route_smem > 48 * 1024) {
    cudaError_t err = cudaFuncSetAttribute(moe_route_kernel<elem_t>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)route_smem);
    if (err != cudaSuccess) return fail(ERB_ERR_CUDA, "moe_route: %s", cudaGetErrorString(err));
  }
  if (route_smem > 200 * 1024) return fail(ERB_ERR_UNSUPPORTED, "moe_route: rows of %d entries with %d experts", width, n_experts);
  launch_chained(moe_route_kernel<elem_t>, dim3((n_tokens + kRouteTokens - 1) / kRouteTokens), dim3(kRouteThreads), route_smem, s,
                 (const elem_t*)x, ld, w_router, n_tokens, width, n_experts, top, choice, score, score_kind, n_groups, keep_groups);
  int rc = check_launch("moe_route");
  if (rc) return rc;
  launch_chained(moe_lists_kernel, dim3(n_experts), dim3(256), sizeof(int) * n_experts, s, (const int*)choice, n_pairs, n_experts,
                 tile_rows > 0 ? tile_rows : kTM, counts, offsets, tiles, order);
  return check_launch("moe_lists");
}

// mode 1 (gated): act[list row][n_out] = silu(gate) * up from x (gathered, scaled by `score` if given); mode 2 (single):
// act[list row][n_out] = relu(up)^2 from x; mode 0 (down): parts[choice][token][n_out] from act rows, times `score` if given.
ERB_EXPORT int erb_moe_product(const void* a, int lda, const void* weights, const int* offsets, const int* tiles,
                               const int* order, const float* score, int n_experts, int top, int n_tokens, int n_out, int k_dim,
                               int mode, void* act, float* parts, void* stream) {
  if (n_tokens <= 0) return ERB_OK;
  if (n_out <= 0 || k_dim <= 0 || n_experts <= 0 || top <= 0 || mode < 0 || mode > 2) return fail(ERB_ERR_ARG, "moe_product: bad sizes");
  const int max_tiles = (n_tokens * top + kTM - 1) / kTM + n_experts;
  dim3 grid(max_tiles, (n_out + kTN - 1) / kTN);
  if (mode == ERB_MOE_SINGLE)
    launch_chained(moe_product_kernel<elem_t, ERB_MOE_SINGLE>, grid, dim3(256), 0, (cudaStream_t)stream, (const elem_t*)a, lda,
                   (const elem_t*)weights, offsets, tiles, order, score, n_experts, top, n_tokens, n_out, k_dim, (elem_t*)act,
                   parts);
  else if (mode == ERB_MOE_GATED)
    launch_chained(moe_product_kernel<elem_t, ERB_MOE_GATED>, grid, dim3(256), 0, (cudaStream_t)stream, (const elem_t*)a, lda,
                   (const elem_t*)weights, offsets, tiles, order, score, n_experts, top, n_tokens, n_out, k_dim, (elem_t*)act,
                   parts);
  else
    launch_chained(moe_product_kernel<elem_t, ERB_MOE_DOWN>, grid, dim3(256), 0, (cudaStream_t)stream, (const elem_t*)a, lda,
                   (const elem_t*)weights, offsets, tiles, order, score, n_experts, top, n_tokens, n_out, k_dim, (elem_t*)act,
                   parts);
  return check_launch("moe_product");
}
