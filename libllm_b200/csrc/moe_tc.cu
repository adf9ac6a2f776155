// The experts' products of a routed feed-forward on the 5th-generation tensor cores.
//
// Rows (token, choice) lie sorted by expert (csrc/moe.cu: moe_sort_kernel gives offsets, the
// permutation and a table of token tiles, each within one expert).  Both products of all experts
// are one launch each of a persistent kernel built like the dense product (csrc/gemm_tc.cu):
// an expert's weight rows are the 128-row operand of tcgen05.mma and a tile of TN sorted rows its N
// operand; one warp issues TMA loads (128-byte swizzle) of [64 x 64 k] boxes of the stacked weights
// [experts * rows, K] and a [TN x 64 k] box of the sorted activations into a ring of stages, one warp
// issues the products into one of two accumulators in tensor memory, four warps read the other
// accumulator and store.  The tiles are not known to the host: every CTA reads their number from
// the table and walks tile = CTA, CTA + grid, ...; tile -> (token tile, 128 weight rows).
//
//   first product   A = the tokens' rows gathered into sorted order (csrc/moe.cu: moe_gather_kernel),
//                   W = up [experts, ff, width]; the epilogue applies the row's weight and the
//                   activation (csrc/moe.cu has the rule) and stores bfloat16 mid[place, ff].
//   second product  A = mid, W = down [experts, width, ff]; the epilogue scatters 32-bit rows to
//                   out[choice][token].
// Gated experts (csrc/moe.cu has the layout: rows of gate and up interleaved, N = 2 ff): a lane of the first
// epilogue holds one weight row, so neighbouring lanes hold a feature's gate and up values for the same token;
// the even lane takes its neighbour's by a shuffle and stores weight * act(gate) * up to mid[place, feature].
// A box of sorted rows may reach into the next expert's rows, and a box of weight rows into the next
// expert's: such products are computed and never stored.  Every wait has a time limit, after which
// the CTA records a code in `status`, lets its loads land, frees its tensor memory and returns.
#include "common.cuh"
#include "tc_common.cuh"
#include <math.h>

LLM_DEFINE_LAST_ERROR(llm_moe_tc_last_error)

namespace {

constexpr int MT_THREADS = 192;
constexpr int MT_ROWS = 128;
constexpr int MT_A_BYTES = MT_ROWS * TC_BK * 2;

template <int KIND>
__device__ __forceinline__ float mt_activate(float z) {
  if (KIND == 0) return 0.5f * z * (1.f + erff(z * 0.70710678118654752f));
  if (KIND == 1) return 0.5f * z * (1.f + tanhf(0.79788456080286536f * (z + 0.044715f * z * z * z)));
  if (KIND == 3) return z > 0.f ? z * z : 0.f;
  return z / (1.f + expf(-z));
}

template <int TN>
struct MtShape {
  static constexpr int B_BYTES = TN * TC_BK * 2;
  static constexpr int STAGE_BYTES = MT_A_BYTES + B_BYTES;
  static constexpr int BUDGET = TN <= 32 ? 100 * 1024 : 192 * 1024;
  static constexpr int STAGES = BUDGET / STAGE_BYTES;
  static constexpr int TMEM_COLS = 2 * TN < 32 ? 32 : 2 * TN;
  static constexpr size_t SMEM = 1024 + (size_t)STAGES * STAGE_BYTES + 256;
};

// ACT: the activation of the first product (csrc/moe.cu numbers them), or -1 for the second product.  The kind of
// product and the activation are the compiler's to know: with them as arguments the epilogue's loop was
// branches around every element, and the sixteen values of a load were worked through one after the other.
template <int TN, int ACT, bool GATED>
__global__ void __launch_bounds__(MT_THREADS, 1)
moe_tc_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, int N, int K,
              const int *__restrict__ offsets, const int *__restrict__ perm, const int *__restrict__ tiles,
              const float *__restrict__ weight, int n_tokens, int top, int weight_on,
              __nv_bfloat16 *__restrict__ mid, float *__restrict__ out, int *status) {
  using S = MtShape<TN>;
  constexpr int STAGES = S::STAGES;
  constexpr bool SECOND = ACT < 0;
  extern __shared__ unsigned char smem_raw[];
  unsigned char *smem = (unsigned char *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  unsigned long long *bars = (unsigned long long *)(smem + (size_t)STAGES * S::STAGE_BYTES);
  const unsigned bar_full = smem_u32(bars), bar_empty = smem_u32(bars + STAGES);
  const unsigned bar_tfull = smem_u32(bars + 2 * STAGES), bar_tempty = smem_u32(bars + 2 * STAGES + 2);
  unsigned *tmem_slot = (unsigned *)(bars + 2 * STAGES + 4);
  volatile int *abort_flag = (volatile int *)(tmem_slot + 1);

  const int warp = __shfl_sync(0xffffffffu, threadIdx.x >> 5, 0), lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(bar_full + 8 * s, 1);
      mbar_init(bar_empty + 8 * s, 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(bar_tfull + 8 * a, 1);
      mbar_init(bar_tempty + 8 * a, 4);
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_x) : "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "r"((unsigned)S::TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const unsigned tmem_base = *tmem_slot;

  // The table of token tiles is written by the sort kernel, two launches back.  The kernel is launched without the
  // overlap attribute: it starts when everything before it in the stream is complete, and what follows it starts
  // when it is.
  grid_dependency_wait();
  const int row_tiles = (N + MT_ROWS - 1) / MT_ROWS;
  const int n_tiles = tiles[0] * row_tiles;
  const int n_kblocks = (K + TC_BK - 1) / TC_BK;

  if (warp == 0) {
    // ------------------------------------------------------------ loader
    const bool leader = elect_one();
    int stage = 0;
    unsigned phase = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
      const int tt = tile / row_tiles, row_tile = tile - tt * row_tiles;
      const int expert = tiles[1 + 2 * tt], place0 = tiles[2 + 2 * tt];
      const int w_row = expert * N + row_tile * MT_ROWS;
      for (int kb = 0; kb < n_kblocks; ++kb) {
        ok = __all_sync(0xffffffffu, mbar_wait(bar_empty + 8 * stage, phase ^ 1, abort_flag, status, 41));
        if (!ok) break;
        if (leader) {
          const unsigned dst = smem_u32(smem + (size_t)stage * S::STAGE_BYTES);
          mbar_expect_tx(bar_full + 8 * stage, S::STAGE_BYTES);
          tma_load_2d(dst, &map_w, kb * TC_BK, w_row, bar_full + 8 * stage);
          tma_load_2d(dst + MT_A_BYTES / 2, &map_w, kb * TC_BK, w_row + 64, bar_full + 8 * stage);
          tma_load_2d(dst + MT_A_BYTES, &map_x, kb * TC_BK, place0, bar_full + 8 * stage);
        }
        if (++stage == STAGES) {
          stage = 0;
          phase ^= 1;
        }
      }
    }
    if (leader && (!ok || *abort_flag)) {
      const unsigned long long t0 = globaltimer();
      for (int s = 0; s < STAGES; ++s)
        while (!mbar_try(bar_full + 8 * s, 0) && !mbar_try(bar_full + 8 * s, 1) && globaltimer() - t0 < 2000000ull) {
        }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ tensor-core issue
    const bool leader = elect_one();
    constexpr unsigned IDESC = instr_desc(MT_ROWS, TN);
    int stage = 0;
    unsigned phase = 0;
    int iter = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x, ++iter) {
      const int acc = iter & 1;
      const unsigned acc_phase = (iter >> 1) & 1;
      ok = __all_sync(0xffffffffu, mbar_wait(bar_tempty + 8 * acc, acc_phase ^ 1, abort_flag, status, 42));
      if (!ok) break;
      tc_fence_after();
      const unsigned d_tmem = tmem_base + acc * TN;
      for (int kb = 0; kb < n_kblocks; ++kb) {
        ok = __all_sync(0xffffffffu, mbar_wait(bar_full + 8 * stage, phase, abort_flag, status, 43));
        if (!ok) break;
        tc_fence_after();
        const unsigned a_addr = smem_u32(smem + (size_t)stage * S::STAGE_BYTES);
        const unsigned long long a_desc = smem_desc(a_addr), b_desc = smem_desc(a_addr + MT_A_BYTES);
        if (leader) {
#pragma unroll
          for (int kk = 0; kk < TC_BK / 16; ++kk)
            tc_mma(d_tmem, a_desc + (unsigned long long)(kk * 2), b_desc + (unsigned long long)(kk * 2), IDESC,
                   (kk > 0 || kb > 0) ? 1u : 0u);
          tc_commit(bar_empty + 8 * stage);
        }
        __syncwarp();
        if (++stage == STAGES) {
          stage = 0;
          phase ^= 1;
        }
      }
      if (ok && leader) tc_commit(bar_tfull + 8 * acc);
      __syncwarp();
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..5)
    const int quarter = warp & 3;
    int iter = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x, ++iter) {
      const int tt = tile / row_tiles, row_tile = tile - tt * row_tiles;
      const int expert = tiles[1 + 2 * tt], place0 = tiles[2 + 2 * tt];
      const int count = min(TN, offsets[expert + 1] - place0);
      // The tile's rows: where each one's result goes and its weight, a row to a lane (asked for before the
      // accumulator is waited for, handed round by shuffles in the loop: no load stands between two stores).
      int my_row[TN / 32];
      float my_w[TN / 32];
#pragma unroll
      for (int j = 0; j < TN / 32; ++j) {
        const int tok = j * 32 + lane;
        const int id = tok < count ? perm[place0 + tok] : 0;
        my_w[j] = tok < count ? weight[id] : 0.f;
        my_row[j] = SECOND ? (id % top) * n_tokens + id / top : place0 + tok;
      }
      const int acc = iter & 1;
      const unsigned acc_phase = (iter >> 1) & 1;
      ok = __all_sync(0xffffffffu, mbar_wait(bar_tfull + 8 * acc, acc_phase, abort_flag, status, 44));
      if (!ok) break;
      tc_fence_after();
      const int f = row_tile * MT_ROWS + quarter * 32 + lane;       // the weight row = output feature
#pragma unroll
      for (int c0 = 0; c0 < TN; c0 += 16) {
        if (c0 < count) {                                            // the same in all lanes
          float v[16];
          tc_ld16(tmem_base + ((unsigned)(quarter * 32) << 16) + (unsigned)(acc * TN + c0), v);
          // all sixteen values first, then their stores: the values do not wait for one another
          float y[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            if (SECOND) {
              y[i] = v[i];
            } else if (GATED) {
              const float w = __shfl_sync(0xffffffffu, my_w[c0 >> 5], (c0 & 31) + i);
              const float other = __shfl_xor_sync(0xffffffffu, v[i], 1);     // the odd lane's value: the up row
              y[i] = w * (mt_activate<SECOND ? 0 : ACT>(v[i]) * other);
            } else {
              const float w = __shfl_sync(0xffffffffu, my_w[c0 >> 5], (c0 & 31) + i);
              const float a = mt_activate<SECOND ? 0 : ACT>(weight_on == 0 ? w * v[i] : v[i]);
              y[i] = weight_on == 0 ? a : w * a;
            }
          }
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const int row = __shfl_sync(0xffffffffu, my_row[c0 >> 5], (c0 & 31) + i);
            if (c0 + i < count && f < N) {
              if (SECOND) out[(size_t)row * N + f] = y[i];
              else if (!GATED) mid[(size_t)row * N + f] = __float2bfloat16_rn(y[i]);
              else if ((lane & 1) == 0) mid[(size_t)row * (N / 2) + f / 2] = __float2bfloat16_rn(y[i]);
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_tempty + 8 * acc);
    }
  }

  // ---------------------------------------------------------------- teardown
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    __syncwarp();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((unsigned)S::TMEM_COLS)
                 : "memory");
  }
}

template <int TN, int ACT, bool GATED>
int launch_moe_tc(const void *a, long long n_rows, const void *w, int n_experts, int N, int K, const int *offsets,
                  const int *perm, const int *tiles, const float *weight, int n_tokens, int top, int weight_on, void *mid,
                  float *out, int *status, cudaStream_t stream) {
  using S = MtShape<TN>;
  CUtensorMap map_w, map_x;
  int rc = get_map(w, (long long)n_experts * N, K, K, 64, &map_w);
  if (rc != LLM_OK) return rc;
  rc = get_map(a, n_rows, K, K, TN, &map_x);
  if (rc != LLM_OK) return rc;
  auto kern = moe_tc_kernel<TN, ACT, GATED>;
  LLM_CHECK_CUDA(llm_allow_smem(kern, S::SMEM), "moe_tc attribute");
  const long long most = ((long long)(n_experts < n_rows ? n_experts : n_rows) + n_rows / TN) * ((N + MT_ROWS - 1) / MT_ROWS);
  const int grid = (int)(most < sm_count() ? most : sm_count());
  LLM_CHECK_CUDA(llm_launch_after(kern, dim3(grid), dim3(MT_THREADS), S::SMEM, stream, map_w, map_x, N, K, offsets, perm, tiles, weight,
                            n_tokens, top, weight_on, (__nv_bfloat16 *)mid, out, status),
                 "moe_tc launch");
  return LLM_OK;
}

}  // namespace

// Rows of a token tile of the table that the products of `n_rows` rows want (moe_sort's tile_rows).
LLM_EXPORT int llm_moe_tc_tile_rows(int n_rows) { return n_rows <= 512 ? 32 : 128; }
LLM_EXPORT int llm_moe_tc_supports(int width, int ff) { return width % 8 == 0 && ff % 8 == 0; }

// xs [tokens * top, width] bfloat16: the tokens' rows in sorted order; up [experts, ff, width], down
// [experts, width, ff]; mid [tokens * top, ff] bfloat16 scratch; out [top, tokens, width] 32-bit.  The table
// `tiles` must have been made with tiles of llm_moe_tc_tile_rows(tokens * top) rows.
LLM_EXPORT int llm_moe_tc(const void *xs, const void *up, const void *down, const int *offsets, const int *perm,
                          const int *tiles, const float *weight, int n_tokens, int n_experts, int top, int width, int ff,
                          int act, int weight_on, int gated, void *mid, float *out, int *status, cudaStream_t stream) {
  if (n_tokens == 0) return LLM_OK;
  LLM_REQUIRE(!gated || weight_on == 1, "moe_tc: gated experts take their weight on the output");
  LLM_REQUIRE(n_tokens > 0 && top > 0 && width > 0 && ff > 0 && n_experts > 0, "moe_tc: bad sizes");
  LLM_REQUIRE(llm_moe_tc_supports(width, ff), "moe_tc: widths %d / %d must be multiples of 8", width, ff);
  LLM_REQUIRE((uintptr_t)xs % 16 == 0 && (uintptr_t)up % 16 == 0 && (uintptr_t)down % 16 == 0 && (uintptr_t)mid % 16 == 0,
              "moe_tc: operands must be 16-byte aligned");
  LLM_REQUIRE((long long)n_experts * (2 * ff > width ? 2 * ff : width) < (1ll << 31), "moe_tc: the stacked weights have too many rows");
  LLM_REQUIRE(act >= 0 && act <= 3, "moe_tc: unknown activation %d", act);
  const long long n_rows = (long long)n_tokens * top;
#define MT_FIRST(TN, ACT, GATED)                                                                                             \
  launch_moe_tc<TN, ACT, GATED>(xs, n_rows, up, n_experts, GATED ? 2 * ff : ff, width, offsets, perm, tiles, weight, n_tokens, top, \
                                weight_on, mid, nullptr, status, stream)
#define MT_ACTS(TN, GATED) (act == 0 ? MT_FIRST(TN, 0, GATED) : act == 1 ? MT_FIRST(TN, 1, GATED) : act == 2 ? MT_FIRST(TN, 2, GATED) : MT_FIRST(TN, 3, GATED))
#define MT_BOTH(TN)                                                                                                          \
  do {                                                                                                                       \
    const int rc = gated ? MT_ACTS(TN, true) : MT_ACTS(TN, false);                                                           \
    if (rc != LLM_OK) return rc;                                                                                             \
    return launch_moe_tc<TN, -1, false>(mid, n_rows, down, n_experts, width, ff, offsets, perm, tiles, weight, n_tokens, top, \
                                        weight_on, nullptr, out, status, stream);                                            \
  } while (0)
  if (llm_moe_tc_tile_rows((int)n_rows) == 32) MT_BOTH(32);
  MT_BOTH(128);
#undef MT_BOTH
#undef MT_ACTS
#undef MT_FIRST
}
