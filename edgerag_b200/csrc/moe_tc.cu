// The routed experts' products on the 5th-generation tensor cores (bfloat16 operands, float accumulation).
//
// The router's kernels leave, on the device, every expert's list of (token, choice) pairs with offsets, and the offsets
// in row tiles of `tile_rows` rows.  A block here owns one row tile of one expert's list (up to MT rows, MT = tile_rows)
// and 256 rows of that expert's weight, as two accumulators of 128 rows each:
//
//   gather      (a kernel of its own, before the gate/up product) writes the rows of the lists once, in list order:
//               xs[list row] = round(score * x[token]), so that both products read their rows as plain 2-d tiles
//   warp 0      one thread brings tiles of the weight (2 x 128 rows x 64 k) and of the rows (MT x 64 k) into
//               128-byte-swizzled shared memory with TMA tensor copies, five stages deep (tiles of 128 rows: two, and two
//               blocks share an SM)
//   warp 1      one thread issues tcgen05.mma with the weight's rows as the M = 128 side and the list's rows as the N side,
//               once per accumulator; the accumulators are 2 x MT columns of TMEM
//   all warps   read the accumulators (a thread = a row of the weight in each) and finish from registers:
//               gate/up: the first accumulator holds 128 gate rows, the second the 128 up rows that go with them:
//                        act[list row][column] = silu(gate) * up;
//               down:    parts[choice][token][column] = the float sums (columns n0 + thread and n0 + 128 + thread),
//                        one partial result per choice of a token, times the pair's score where the expert's output
//                        (not its input) carries the weight;
//               single:  one product without a gate branch, act[list row][column] = relu(sum)^2 for both accumulators
//
// A tile's rows past the end of its expert's list are rows of the next expert (or nothing): they are multiplied along and
// never stored.  A tile of weight rows past the expert's last row reads the next expert's rows: not stored either.  k is
// walked in one order whatever tile a row falls into, and a row is a column of the accumulator that no other row touches,
// so a token's result does not depend on the other tokens of the step.
//
// Every wait is bounded; a thread that gives up raises a block-wide flag, the block lets its copies land, records
// 5000000 + block in *status (if given), frees its TMEM and writes nothing.
#include <stdarg.h>
#include <stdio.h>

#undef ERB_ELEM
#define ERB_ELEM 1
#include "tc_common.cuh"

using namespace erb;

ERB_DEFINE_LAST_ERROR(erb_last_error)

namespace {

constexpr int kTileN = 128;              // rows of the weight per block (the M side of the instruction)
constexpr int kTileK = 64;               // k per stage: one 128-byte swizzle span
constexpr int kThreads = 128;
constexpr uint32_t kWBytes = kTileN * kTileK * 2;      // 16 KB

template <int MT> struct Plan {
  static constexpr uint32_t kABytes = MT * kTileK * 2;
  static constexpr uint32_t kStageBytes = 2 * kWBytes + kABytes;
  // tiles of 128 rows: two stages a block, so that two blocks share an SM and one's epilogue runs under the other's products
  static constexpr int kStages = MT >= 128 ? 2 : 5;
  static constexpr uint32_t kSmemBytes = kStages * kStageBytes + 1024;
  static constexpr uint32_t kTmemCols = 2 * MT < 32 ? 32 : 2 * MT;
};

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar) : "memory");
}

// xs[list row][:] = round(score[pair] * x[pair / top][:]) for every row of the lists; 8 values a thread.
__global__ void __launch_bounds__(256)
moe_gather_kernel(const __nv_bfloat16* __restrict__ x, int ldx, const int* __restrict__ order, const float* __restrict__ score,
                  int top, int n_pairs, int width, __nv_bfloat16* __restrict__ xs) {
  chain_wait();
  const int per_row = width / 8;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < (long long)n_pairs * per_row;
       idx += (long long)gridDim.x * blockDim.x) {
    const int row = (int)(idx / per_row), c = (int)(idx % per_row);
    const int pair = order[row];
    const float s = score ? score[pair] : 1.f;
    const uint4 raw = *reinterpret_cast<const uint4*>(x + (size_t)(pair / top) * ldx + c * 8);
    const __nv_bfloat16* in = reinterpret_cast<const __nv_bfloat16*>(&raw);
    uint4 packed;
    __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(&packed);
#pragma unroll
    for (int i = 0; i < 8; ++i) o[i] = __float2bfloat16_rn(s * __bfloat162float(in[i]));
    *reinterpret_cast<uint4*>(xs + (size_t)row * width + c * 8) = packed;
  }
}

// grid (row tiles of the lists: an upper bound, column tiles of the weight).  GATED: the weight of an expert holds n_out
// gate rows and then n_out up rows, a tile takes 128 of each; else it takes 256 neighbouring rows.
constexpr int kDown = 0, kGated = 1, kSingle = 2;
template <int MT, int MODE>
__global__ void __launch_bounds__(kThreads, MT >= 128 ? 2 : 1)
moe_tc_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_a,
              const int* __restrict__ offsets, const int* __restrict__ tiles, const int* __restrict__ order, int n_experts,
              int top, int n_tokens, int n_out, int K, __nv_bfloat16* __restrict__ act, float* __restrict__ parts,
              const float* __restrict__ out_score, int* __restrict__ status) {
  constexpr bool GATED = MODE == kGated, PAIRS = MODE == kDown;
  using P = Plan<MT>;
  constexpr int kStages = P::kStages;
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bars[2 * kStages + 1];      // full, empty, accumulator done
  __shared__ int s_abort;
  __shared__ uint32_t tmem_slot;
  __shared__ int pair_s[MT];
  chain_wait();                                                 // the lists and the rows come from the kernels before
  const int tile = blockIdx.x;
  if (tile >= tiles[n_experts]) return;                         // (before anything is set up: nothing to give back)
  int e = 0;
  {
    int lo = 0, hi = n_experts;                                 // the last e with tiles[e] <= tile
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (tiles[mid] <= tile) lo = mid; else hi = mid;
    }
    e = lo;
  }
  const int row0 = offsets[e] + (tile - tiles[e]) * MT;
  const int n_rows = min(MT, offsets[e + 1] - row0);
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (base - raw);
  const uint32_t full0 = smem_u32(&bars[0]), empty0 = smem_u32(&bars[kStages]), done_bar = smem_u32(&bars[2 * kStages]);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n0 = blockIdx.y * (GATED ? kTileN : 2 * kTileN);    // first output column of this block
  const int w_row0 = e * (GATED ? 2 : 1) * n_out + n0;          // its first row in the stacked weights
  const int n_kb = (K + kTileK - 1) / kTileK;

  auto ask = [&](int i) {
    const int s = i % kStages;
    mbar_expect(full0 + 8 * s, 2 * kWBytes + P::kABytes);
    const uint32_t dst = base + s * P::kStageBytes;
    tma_load_2d(dst, &map_w, i * kTileK, w_row0, full0 + 8 * s);
    tma_load_2d(dst + kWBytes, &map_w, i * kTileK, w_row0 + (GATED ? n_out : kTileN), full0 + 8 * s);
    tma_load_2d(dst + 2 * kWBytes, &map_a, i * kTileK, row0, full0 + 8 * s);
  };
  const int ahead = min(kStages, n_kb);
  if (tid == 0) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_a) : "memory");
    for (int s = 0; s < kStages; ++s) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
    mbar_init(done_bar, 1);
    s_abort = 0;
    mbar_init_fence();
    for (int i = 0; i < ahead; ++i) ask(i);
  }
  if (PAIRS && tid < MT) pair_s[tid] = tid < n_rows ? order[row0 + tid] : -1;
  if (PAIRS && MT > kThreads) {
    for (int r = kThreads + tid; r < MT; r += kThreads) pair_s[r] = r < n_rows ? order[row0 + r] : -1;
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)), "r"(P::kTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  const uint32_t tmem = tmem_slot;
  volatile int* abort_flag = &s_abort;
  int asked = tid == 0 ? ahead : 0;     // stages the copy thread has asked for

  if (warp == 0 && lane == 0) {
    for (int i = ahead; i < n_kb; ++i) {
      if (!mbar_wait_or_abort(empty0 + 8 * (i % kStages), ((i / kStages) - 1) & 1, abort_flag)) break;
      ask(i);
      asked = i + 1;
    }
  } else if (warp == 1 && lane == 0) {
    constexpr uint32_t idesc = mma_idesc(kTileN, MT, false);
    bool ok = true;
    for (int i = 0; i < n_kb && ok; ++i) {
      const int s = i % kStages;
      ok = mbar_wait_or_abort(full0 + 8 * s, (i / kStages) & 1, abort_flag);
      if (!ok) break;
      fence_after_sync();
      const uint32_t st = base + s * P::kStageBytes;
      const uint64_t dw0 = make_desc(st), dw1 = make_desc(st + kWBytes), da = make_desc(st + 2 * kWBytes);
#pragma unroll
      for (int k = 0; k < kTileK / 16; ++k) {
        mma_bf16(tmem, dw0 + 2 * k, da + 2 * k, idesc, (i > 0 || k > 0) ? 1u : 0u);
        mma_bf16(tmem + MT, dw1 + 2 * k, da + 2 * k, idesc, (i > 0 || k > 0) ? 1u : 0u);
      }
      mma_commit(empty0 + 8 * s);
    }
    if (ok) mma_commit(done_bar);
  }
  // ---- the accumulator: lane = row of the weight, column = row of the list ----
  bool ok = true;
  if (lane == 0) ok = mbar_wait_or_abort(done_bar, 0, abort_flag);
  ok = __all_sync(0xffffffffu, ok) != 0;
  __syncthreads();
  if (*abort_flag) {
    if (tid == 0) {
      for (int i = max(0, asked - kStages); i < asked; ++i) mbar_wait(full0 + 8 * (i % kStages), (i / kStages) & 1);
      if (status) atomicCAS(status, 0, 5000000 + (int)blockIdx.x);
    }
    __syncthreads();
    if (warp == 1) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(P::kTmemCols) : "memory");
    return;
  }
  // ---- finishing, from registers: thread = a row of the weight in each accumulator = an output column ----
  fence_after_sync();
  {
    const uint32_t t_lane = tmem + ((uint32_t)(warp * 32) << 16);
    const int n_a = n0 + tid, n_b = n0 + kTileN + tid;          // (gated: one column n_a from both accumulators)
#pragma unroll 1
    for (int c = 0; c < MT / 16; ++c) {
      if (16 * c >= n_rows) break;                              // (the same for every thread: the loads are collective)
      float v0[16], v1[16];
      tmem_ld16(t_lane + 16 * c, v0);
      tmem_ld16(t_lane + MT + 16 * c, v1);
      tmem_ld_wait();
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const int m = 16 * c + i;
        if (m >= n_rows) break;
        if (GATED) {
          if (n_a < n_out) act[(size_t)(row0 + m) * n_out + n_a] = __float2bfloat16_rn(silu_mul(v0[i], v1[i]));
        } else if (MODE == kSingle) {
          const float za = fmaxf(v0[i], 0.f), zb = fmaxf(v1[i], 0.f);
          if (n_a < n_out) act[(size_t)(row0 + m) * n_out + n_a] = __float2bfloat16_rn(za * za);
          if (n_b < n_out) act[(size_t)(row0 + m) * n_out + n_b] = __float2bfloat16_rn(zb * zb);
        } else {
          const int pair = pair_s[m];
          const float sc = out_score ? out_score[pair] : 1.f;
          float* dst = parts + ((size_t)(pair % top) * n_tokens + pair / top) * n_out;
          if (n_a < n_out) dst[n_a] = v0[i] * sc;
          if (n_b < n_out) dst[n_b] = v1[i] * sc;
        }
      }
    }
  }
  fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    fence_after_sync();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(P::kTmemCols) : "memory");
  }
}

// A tensor map over rows of 64-k boxes: matrix[rows][K] with row stride ld, boxes of box_rows rows.
int matrix_map(CUtensorMap* out, const void* p, long long rows, int K, int ld, int box_rows) {
  static std::map<std::tuple<const void*, long long, int, int, int>, CUtensorMap> maps;
  static std::mutex mutex;
  std::lock_guard<std::mutex> lock(mutex);
  const auto key = std::make_tuple(p, rows, K, ld, box_rows);
  auto it = maps.find(key);
  if (it == maps.end()) {
    CUtensorMap m;
    const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    const cuuint32_t box[2] = {(cuuint32_t)kTileK, (cuuint32_t)box_rows};
    const cuuint32_t elem[2] = {1, 1};
    const CUresult r = cuTensorMapEncodeTiled(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(p), dims, strides, box, elem,
                                              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                              CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(ERB_ERR_CUDA, "moe_tc: cuTensorMapEncodeTiled failed (%d)", (int)r);
    if (maps.size() > 8192) maps.clear();
    it = maps.emplace(key, m).first;
  }
  *out = it->second;
  return ERB_OK;
}

template <int MT, int MODE>
int launch(const CUtensorMap& mw, const CUtensorMap& ma, const int* offsets, const int* tiles, const int* order, int n_experts,
           int top, int n_tokens, int n_out, int K, void* act, float* parts, const float* out_score, int* status,
           cudaStream_t stream) {
  constexpr bool GATED = MODE == kGated;
  auto kern = moe_tc_kernel<MT, MODE>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Plan<MT>::kSmemBytes);
    if (e != cudaSuccess) return fail(ERB_ERR_CUDA, "moe_tc: %s", cudaGetErrorString(e));
    configured = true;
  }
  const long long pairs = (long long)n_tokens * top;
  const int per_tile = GATED ? kTileN : 2 * kTileN;
  // an upper bound of the row tiles: every expert's last tile may be short
  const dim3 grid((unsigned)((pairs + MT - 1) / MT + n_experts), (unsigned)((n_out + per_tile - 1) / per_tile));
  launch_chained(kern, grid, dim3(kThreads), Plan<MT>::kSmemBytes, stream, mw, ma, offsets, tiles, order, n_experts, top, n_tokens,
                 n_out, K, (__nv_bfloat16*)act, parts, out_score, status);
  return check_launch("moe_tc");
}

template <int MODE>
int run(const void* a, const void* w, const int* offsets, const int* tiles, const int* order, int n_experts, int top, int n_tokens,
        int n_out, int K, int tile_rows, void* act, float* parts, const float* out_score, int* status, cudaStream_t stream) {
  constexpr bool GATED = MODE == kGated;
  if (n_tokens <= 0) return ERB_OK;
  if (n_out <= 0 || K <= 0 || n_experts <= 0 || top <= 0) return fail(ERB_ERR_ARG, "moe_tc: bad sizes");
  if ((K & 7) || ((uintptr_t)a & 15) || ((uintptr_t)w & 15))
    return fail(ERB_ERR_UNSUPPORTED, "moe_tc: k must be a multiple of 8, operands 16-byte aligned");
  const long long pairs = (long long)n_tokens * top, w_rows = (long long)n_experts * (GATED ? 2 : 1) * n_out;
  if (pairs > 0x7fffffffLL || w_rows > 0x7fffffffLL) return fail(ERB_ERR_UNSUPPORTED, "moe_tc: too many rows");
  CUtensorMap mw, ma;
  int rc;
  if ((rc = matrix_map(&mw, w, w_rows, K, K, kTileN)) || (rc = matrix_map(&ma, a, pairs, K, K, tile_rows))) return rc;
#define ERB_MOE_CASE(MT) \
  case MT: return launch<MT, MODE>(mw, ma, offsets, tiles, order, n_experts, top, n_tokens, n_out, K, act, parts, out_score, status, stream);
  switch (tile_rows) {
    ERB_MOE_CASE(16)
    ERB_MOE_CASE(32)
    ERB_MOE_CASE(64)
    ERB_MOE_CASE(128)
    default: return fail(ERB_ERR_ARG, "moe_tc: tiles of %d rows (takes 16, 32, 64, 128)", tile_rows);
  }
#undef ERB_MOE_CASE
}

}  // namespace

// xs[list row][width] = round(score[pair] * x[token of pair][:]), pair = order[list row]; bfloat16, width a multiple of 8,
// rows 16-byte aligned.
ERB_EXPORT int erb_moe_tc_gather(const void* x, int ldx, const int* order, const float* score, int top, int n_tokens, int width,
                                 void* xs, void* stream) {
  if (n_tokens <= 0) return ERB_OK;
  if (width <= 0 || (width & 7) || (ldx & 7) || ((uintptr_t)x & 15) || ((uintptr_t)xs & 15) || top <= 0)
    return fail(ERB_ERR_UNSUPPORTED, "moe_tc_gather: rows must be multiples of 8 entries and 16-byte aligned");
  const long long work = (long long)n_tokens * top * (width / 8);
  const unsigned blocks = (unsigned)((work + 255) / 256 < 4096 ? (work + 255) / 256 : 4096);
  launch_chained(moe_gather_kernel, dim3(blocks), dim3(256), 0, (cudaStream_t)stream, (const __nv_bfloat16*)x, ldx, order, score, top,
                 n_tokens * top, width, (__nv_bfloat16*)xs);
  return check_launch("moe_tc_gather");
}

// act[list row][ff] = silu(W_gate r) * (W_up r) for the rows r = xs[list row] of every expert's list; w [experts][2 ff][k]
// (gate rows, then up rows).  tile_rows: what the lists' tile offsets were made for (16, 32, 64 or 128).
ERB_EXPORT int erb_moe_tc_gate_up(const void* xs, const void* w, const int* offsets, const int* tiles, const int* order,
                                  int n_experts, int top, int n_tokens, int ff, int K, int tile_rows, void* act, int* status,
                                  void* stream) {
  return run<kGated>(xs, w, offsets, tiles, order, n_experts, top, n_tokens, ff, K, tile_rows, act, nullptr, nullptr, status,
                     (cudaStream_t)stream);
}

// act[list row][ff] = relu(W_up r)^2 for the rows r = xs[list row] of every expert's list; w [experts][ff][k].
ERB_EXPORT int erb_moe_tc_up_act(const void* xs, const void* w, const int* offsets, const int* tiles, const int* order,
                                 int n_experts, int top, int n_tokens, int ff, int K, int tile_rows, void* act, int* status,
                                 void* stream) {
  return run<kSingle>(xs, w, offsets, tiles, order, n_experts, top, n_tokens, ff, K, tile_rows, act, nullptr, nullptr, status,
                      (cudaStream_t)stream);
}

// parts[choice][token][width] (float) = W_down act[list row] (times out_score[pair] where given); w [experts][width][ff].
ERB_EXPORT int erb_moe_tc_down(const void* act, const void* w, const int* offsets, const int* tiles, const int* order,
                               int n_experts, int top, int n_tokens, int width, int K, int tile_rows, float* parts,
                               const float* out_score, int* status, void* stream) {
  if (((uintptr_t)parts & 15)) return fail(ERB_ERR_ARG, "moe_tc_down: parts must be 16-byte aligned");
  return run<kDown>(act, w, offsets, tiles, order, n_experts, top, n_tokens, width, K, tile_rows, nullptr, parts, out_score, status,
                    (cudaStream_t)stream);
}
