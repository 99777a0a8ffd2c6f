// The two products of the routed feed-forward (moe.cu) on tensor cores, bfloat16: tiles of 128 rows of one expert
// times 128 weight rows, mma.sync m16n8k16 with float32 accumulation, operands through a three-stage cp.async
// ring (64 columns of k a stage, 108 KB of shared memory: two blocks a multiprocessor keep about 70 KB of weights
// in flight, which a decode step - every touched expert's weights streamed once - needs to fill the memory pipe).
// Eight warps as 4 x 2: a warp owns 32 of the tile's rows and 64 of its weight rows.  (Four warps on 64 rows, two blocks
// a multiprocessor, kept the tensor pipe 43 % busy with an eighth of the warp slots filled.)
// Steps with few rows per expert (single tokens) take a second instance: tiles of 16 rows - one MMA row tile - and
// four warps side by side on 64 weight rows, four stages, four such blocks a multiprocessor (256 weight rows, one
// block a multiprocessor: the same time; two warps on 128 weight rows: a quarter slower).  Such a step streams every touched expert's weights once
// for a handful of rows, and on the wide tile it was bound by the MMAs spent on empty rows (128-row tiles at batch 64:
// 2 TB/s from a cold cache).  Between 12 and 32 rows per expert on average a third instance has tiles of 32 rows (two MMA
// row tiles a warp, otherwise the small one): with 16-row tiles the experts that got 17 rows or more take a second
// tile each, and a few of those push the grid past the blocks that are resident at once - a second, nearly empty wave.
//   gate_up  the 128 weight rows are 64 gate rows and the 64 up rows of the same activation columns; a warp's
//            eight 8-column tiles are four of gate and the same four of up, so silu(gate) * up happens in the
//            accumulator registers; rows are gathered from the step's tokens by (token, choice) pair.
//   down     the 128 weight rows are output columns; a row's result is multiplied by its pair's routing weight
//            and written as float32 to the pair's row (summed over a token's choices by the combine kernel).
// Rows past a tile's end and columns past the matrices' edges are zero-filled in shared memory.
#include "attention_decode.cuh"
#include "common.cuh"
#include "moe.cuh"

namespace mll {

// WM x WN warps, each on 16 MT rows x 8 NT weight rows; BK columns of k a stage.  Rows of BK + 8 elements: ldmatrix
// without bank conflicts.
template <int MT, int NT, int WM, int WN, int BK, int STAGES>
struct MoeMmaShape {
  static constexpr int BM = 16 * MT * WM, BN = 8 * NT * WN, LD = BK + 8, THREADS = 32 * WM * WN;
  static constexpr size_t SMEM = (size_t)STAGES * (BM + BN) * LD * sizeof(__nv_bfloat16);
};
using MoeMmaWide = MoeMmaShape<2, 8, 4, 2, 64, 3>;   // 128 rows x 128 weight rows: prompts
using MoeMmaSmall = MoeMmaShape<1, 2, 1, 4, 64, 4>;  // 16 rows x 64 weight rows: single tokens
using MoeMmaMedium = MoeMmaShape<2, 2, 1, 4, 64, 4>;  // 32 rows x 64 weight rows: single tokens, 12 to 32 rows an expert

// KIND 0: down; 1: gate_up (silu(gate) * up); 2: up alone with gelu (erf form) - the layout of `down`, rows gathered
// by token, the activation in the accumulators, bfloat16 out by place.
template <int KIND, int MT, int NT, int WM, int WN, int MMA_BK, int MMA_STAGES>
__global__ void __launch_bounds__(32 * WM * WN) moe_mma_kernel(MoeProductArgs a) {
  constexpr bool GATE_UP = KIND == 1;
  constexpr bool GATHER = KIND != 0;
  using Shape = MoeMmaShape<MT, NT, WM, WN, MMA_BK, MMA_STAGES>;
  static_assert(NT % 2 == 0, "a warp's 8-column tiles come in pairs");
  constexpr int BM = Shape::BM, BN = Shape::BN, MMA_LD = Shape::LD, MMA_THREADS = Shape::THREADS;
  const int tile = blockIdx.x;
  if (tile >= a.plan.n_tiles[0]) return;
  extern __shared__ __align__(16) unsigned char moe_smem[];
  typedef __nv_bfloat16 (*ATile)[BM][MMA_LD];
  typedef __nv_bfloat16 (*BTile)[BN][MMA_LD];
  ATile a_s = reinterpret_cast<ATile>(moe_smem);
  BTile b_s = reinterpret_cast<BTile>(moe_smem + (size_t)MMA_STAGES * BM * MMA_LD * sizeof(__nv_bfloat16));
  __shared__ int row_src[BM];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int wm = warp / WN, wn = warp % WN;
  const int g = lane >> 2, t = lane & 3;
  const int e = a.plan.tile_expert[tile], row0 = a.plan.tile_row0[tile];
  const int rows = min(BM, a.plan.offsets[e + 1] - row0);
  const int K = a.k, N = a.n;
  const int n0 = blockIdx.y * (GATE_UP ? BN / 2 : BN);  // first activation column (gate_up) or output column (down)
  if (tid < BM) row_src[tid] = tid < rows ? (GATHER ? a.plan.order[row0 + tid] / a.top : row0 + tid) : -1;
  __syncthreads();
  const __nv_bfloat16* act = (const __nv_bfloat16*)a.a;
  const __nv_bfloat16* w = (const __nv_bfloat16*)a.w + (size_t)e * (GATE_UP ? 2 * N : N) * K;

  auto load = [&](int kt, int stage) {
    const int k0 = kt * MMA_BK;
    for (int c = tid; c < BM * (MMA_BK / 8); c += MMA_THREADS) {
      const int r = c / (MMA_BK / 8), cc = c % (MMA_BK / 8);
      const int src = row_src[r];
      const bool in = src >= 0 && k0 + cc * 8 < K;
      cp_async16_zfill(&a_s[stage][r][cc * 8], act + (in ? (size_t)src * K + k0 + cc * 8 : 0), in);
    }
    for (int c = tid; c < BN * (MMA_BK / 8); c += MMA_THREADS) {
      const int r = c / (MMA_BK / 8), cc = c % (MMA_BK / 8);
      // gate_up: the first half of the rows are gate rows n0 + r, the second half the up rows of the same columns
      const int col = GATE_UP ? n0 + (r % (BN / 2)) : n0 + r;
      const size_t wrow = GATE_UP ? (size_t)(r / (BN / 2)) * N + col : (size_t)col;
      const bool in = col < N && k0 + cc * 8 < K;
      cp_async16_zfill(&b_s[stage][r][cc * 8], w + (in ? wrow * K + k0 + cc * 8 : 0), in);
    }
  };

  float acc[MT][NT][4];
#pragma unroll
  for (int m = 0; m < MT; ++m)
#pragma unroll
    for (int n = 0; n < NT; ++n)
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[m][n][i] = 0.f;

  const int nk = (K + MMA_BK - 1) / MMA_BK;
#pragma unroll
  for (int s = 0; s < MMA_STAGES - 1; ++s) {
    if (s < nk) load(s, s);
    cp_async_commit();
  }
  for (int kt = 0; kt < nk; ++kt) {
    cp_async_wait<MMA_STAGES - 2>();
    __syncthreads();
    if (kt + MMA_STAGES - 1 < nk) load(kt + MMA_STAGES - 1, (kt + MMA_STAGES - 1) % MMA_STAGES);
    cp_async_commit();
    const int stage = kt % MMA_STAGES;
#pragma unroll
    for (int ks = 0; ks < MMA_BK / 16; ++ks) {
      unsigned af[MT][4];
#pragma unroll
      for (int m = 0; m < MT; ++m)
        ldmatrix_x4(af[m], &a_s[stage][wm * 16 * MT + m * 16 + (lane & 7) + (((lane >> 3) & 1) << 3)][ks * 16 + ((lane >> 4) << 3)]);
#pragma unroll
      for (int n = 0; n < NT; n += 2) {
        // the warp's n-th 8-column tile: gate_up: the first NT / 2 are gate, the others up, both at columns
        // wn * 4 NT + (n mod NT / 2) * 8.  Tiles n and n + 1 come with one ldmatrix: they lie 8 rows apart, except
        // where a warp has one gate and one up tile, which lie half the weight rows apart.
        constexpr int HALF = NT / 2;
        const int brow = GATE_UP ? (n / HALF) * (BN / 2) + wn * HALF * 8 + (n % HALF) * 8 : wn * NT * 8 + n * 8;
        const int second = GATE_UP && NT == 2 ? BN / 2 : 8;
        unsigned bf[4];
        ldmatrix_x4(bf, &b_s[stage][brow + (lane & 7) + ((lane >> 4) ? second : 0)][ks * 16 + (((lane >> 3) & 1) << 3)]);
#pragma unroll
        for (int m = 0; m < MT; ++m) {
          mma_16816(acc[m][n], af[m], bf[0], bf[1]);
          mma_16816(acc[m][n + 1], af[m], bf[2], bf[3]);
        }
      }
    }
  }
  cp_async_wait<0>();

#pragma unroll
  for (int m = 0; m < MT; ++m)
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int r = wm * 16 * MT + m * 16 + g + 8 * half;
      if (r >= rows) continue;
      const int place = row0 + r;
      if (GATE_UP) {
        __nv_bfloat16* dst = (__nv_bfloat16*)a.out + (size_t)place * N;
#pragma unroll
        for (int n = 0; n < NT / 2; ++n) {
          const int col = n0 + wn * (NT / 2) * 8 + n * 8 + 2 * t;
          if (col >= N) continue;  // N is even: a pair is inside or outside as a whole
          const float g0 = acc[m][n][2 * half], g1 = acc[m][n][2 * half + 1];
          const float u0 = acc[m][n + NT / 2][2 * half], u1 = acc[m][n + NT / 2][2 * half + 1];
          *reinterpret_cast<__nv_bfloat162*>(dst + col) =
              __floats2bfloat162_rn(g0 / (1.f + __expf(-g0)) * u0, g1 / (1.f + __expf(-g1)) * u1);
        }
      } else if (KIND == 2) {
        __nv_bfloat16* dst = (__nv_bfloat16*)a.out + (size_t)place * N;
#pragma unroll
        for (int n = 0; n < NT; ++n) {
          const int col = n0 + wn * NT * 8 + n * 8 + 2 * t;
          if (col >= N) continue;
          const float u0 = acc[m][n][2 * half], u1 = acc[m][n][2 * half + 1];
          *reinterpret_cast<__nv_bfloat162*>(dst + col) =
              __floats2bfloat162_rn(0.5f * u0 * (1.f + erff(u0 * 0.70710678118654752f)),
                                    0.5f * u1 * (1.f + erff(u1 * 0.70710678118654752f)));
        }
      } else {
        const int pair = a.plan.order[place];
        const float pw = a.pair_weight[pair];
        float* dst = (float*)a.out + (size_t)pair * N;
#pragma unroll
        for (int n = 0; n < NT; ++n) {
          const int col = n0 + wn * NT * 8 + n * 8 + 2 * t;
          if (col >= N) continue;
          *reinterpret_cast<float2*>(dst + col) = make_float2(pw * acc[m][n][2 * half], pw * acc[m][n][2 * half + 1]);
        }
      }
    }
}

template <int KIND, int MT, int NT, int WM, int WN, int BK, int STAGES>
int launch_moe_mma(const MoeProductArgs& a, int max_tiles, cudaStream_t stream) {
  using Shape = MoeMmaShape<MT, NT, WM, WN, BK, STAGES>;
  constexpr bool GATE_UP = KIND == 1;
  auto kernel = moe_mma_kernel<KIND, MT, NT, WM, WN, BK, STAGES>;
  cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Shape::SMEM);
  if (err != cudaSuccess) {
    mll_set_error("moe (mma): cannot reserve %zu bytes of shared memory: %s", Shape::SMEM, cudaGetErrorString(err));
    return (int)err;
  }
  const int per_block = GATE_UP ? Shape::BN / 2 : Shape::BN;
  MLL_LAUNCH((kernel), dim3(max_tiles, (a.n + per_block - 1) / per_block), Shape::THREADS, Shape::SMEM, stream, a);
  MLL_LAUNCH_CHECK();
  return 0;
}

template <int KIND>
int launch_moe_mma_rows(const MoeProductArgs& a, int max_tiles, int tile_rows, cudaStream_t stream) {
  if (tile_rows == MoeMmaWide::BM) return launch_moe_mma<KIND, 2, 8, 4, 2, 64, 3>(a, max_tiles, stream);
  if (tile_rows == MoeMmaSmall::BM) return launch_moe_mma<KIND, 1, 2, 1, 4, 64, 4>(a, max_tiles, stream);
  if (tile_rows == MoeMmaMedium::BM) return launch_moe_mma<KIND, 2, 2, 1, 4, 64, 4>(a, max_tiles, stream);
  mll_set_error("moe (mma): tiles of %d rows (known: %d, %d, %d)", tile_rows, MoeMmaSmall::BM, MoeMmaMedium::BM, MoeMmaWide::BM);
  return -1;
}

}  // namespace mll

// Rows of a tile: the wide instance (small = 0) or one of the two for steps with few rows per expert (1: 16 rows, 2: 32).
MLL_API int mll_moe_mma_rows(int small) {
  return small == 1 ? mll::MoeMmaSmall::BM : (small == 2 ? mll::MoeMmaMedium::BM : mll::MoeMmaWide::BM);
}

// bfloat16 only; rows of 16-byte words on both sides of both products.
MLL_API int mll_moe_mma_supported(int width, int inter) { return width > 0 && inter > 0 && width % 8 == 0 && inter % 8 == 0; }

MLL_API int mll_moe_gate_up_mma(const void* h, const void* w, void* act, const int* order, const int* offsets,
                                const int* tile_expert, const int* tile_row0, const int* n_tiles, int max_tiles,
                                int tile_rows, int width, int inter, int top, int form, cudaStream_t stream) {
  MLL_REQUIRE(form == 0 || form == 1, "moe gate_up (mma): unknown expert form %d", form);
  MLL_REQUIRE(mll_moe_mma_supported(width, inter) && max_tiles > 0 && top > 0, "moe gate_up (mma): sizes %d / %d", width, inter);
  MLL_REQUIRE((inter + 31) / 32 <= 65535, "moe gate_up (mma): %d columns are too many for one launch", inter);
  mll::MoeProductArgs a{h, w, act, nullptr, mll::MoePlan{(int*)order, (int*)offsets, (int*)tile_expert, (int*)tile_row0,
                                                         (int*)n_tiles}, width, inter, top};
  if (form == 1) return mll::launch_moe_mma_rows<2>(a, max_tiles, tile_rows, stream);
  return mll::launch_moe_mma_rows<1>(a, max_tiles, tile_rows, stream);
}

MLL_API int mll_moe_down_mma(const void* act, const void* w, float* y, const float* pair_weight, const int* order,
                             const int* offsets, const int* tile_expert, const int* tile_row0, const int* n_tiles,
                             int max_tiles, int tile_rows, int inter, int width, int top, cudaStream_t stream) {
  MLL_REQUIRE(mll_moe_mma_supported(width, inter) && max_tiles > 0 && top > 0, "moe down (mma): sizes %d / %d", width, inter);
  MLL_REQUIRE((width + 63) / 64 <= 65535, "moe down (mma): %d columns are too many for one launch", width);
  mll::MoeProductArgs a{act, w, y, pair_weight, mll::MoePlan{(int*)order, (int*)offsets, (int*)tile_expert,
                                                             (int*)tile_row0, (int*)n_tiles}, inter, width, top};
  return mll::launch_moe_mma_rows<0>(a, max_tiles, tile_rows, stream);
}
