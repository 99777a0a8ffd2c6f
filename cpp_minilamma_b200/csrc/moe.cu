// A routed feed-forward: every token goes through `top` of E small SwiGLU experts, chosen by a linear router.
//
//   z = W_r h + b_r (float32);  the `top` largest z (ties: the lower index);  weights = softmax over those alone
//   out = sum_j weight_j * W_down,e_j (silu(W_gate,e_j h) * W_up,e_j h)
//
// Nothing about the routing ever reaches the host.  The (token, choice) pairs are sorted by expert on the device
// and cut into tiles of up to MOE_BM rows of one expert; the two products run over that tile list with a grid
// sized for the most tiles there can be (pairs / MOE_BM + E), blocks past the real count leaving at once.  So a
// step's launches depend on its number of tokens alone and a decode step can be captured in a graph.
//
//   route      a block per token: its sixteen warps share the E dot products (float32; for many tokens the logits
//              come from a library product instead), then `top` rounds of a warp-wide arg-max and the softmax
//   sort       one block: counts per expert, their running sums, the tile list, the pairs' places
//   gate_up    tile x 128 activation columns: act[place, n] = silu(gate) * up, rows gathered by token
//   down       tile x 128 output columns: y[pair, :] = weight * (W_down act[place]), float32
//   combine    out[t] = y[t, 0] + ... + y[t, top - 1] (+ another part's output for the same rows), fixed order
//
// The products here are the plain form (a thread per output column, the tile's rows in shared memory, float32
// accumulation in k order); every weight of an expert is read once per tile, which is what a decode step needs.
// They serve float32 and sizes whose rows are no whole 16-byte words; bfloat16 steps take the tensor-core kernels of
// moe_mma.cu for the two products.
#include "common.cuh"
#include "moe.cuh"

namespace mll {

// ---- route ---------------------------------------------------------------------------------------------------- //
// How logits become choices and weights.  all_scores 0: the `top` largest logits (+ bias), softmax over those alone.
// all_scores 1: softmax over every expert; the choice goes by score + bias, the weights are the chosen scores over
// their sum, times `scale`.  gate_out: the router's matrix has one more row behind the experts'; the sigmoid of its
// product with the token goes to gate_out[t] (a per-token gate of another part that reads the same rows).
// all_scores 2: scores = sigmoid of every logit; the experts are cut into `groups` runs of consecutive experts of one
// length, a run is rated by its top two scores added up (by its one score if it holds one expert), and only experts of
// the `groups_kept` best-rated runs can be chosen (ties: the lower run); the weights are the chosen scores over their sum, times `scale`.
struct RouteForm {
  int all_scores;
  float scale;
  float* gate_out;
  int groups, groups_kept;
};

template <typename T>
__global__ void __launch_bounds__(512) moe_route_kernel(const T* __restrict__ h, const float* __restrict__ w,
                                                        const float* __restrict__ bias, const float* __restrict__ logits,
                                                        int* __restrict__ chosen, float* __restrict__ weight,
                                                        int n_tokens, int width, int n_experts, int top, RouteForm form) {
  extern __shared__ float z[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int t = blockIdx.x;
  const int n_rows = n_experts + (form.gate_out ? 1 : 0);  // the router's rows, and the row of a per-token gate behind them
  const bool add_bias = bias && !form.all_scores;          // with scores over all experts the bias corrects the choice instead
  if (logits) {  // w h was formed elsewhere
    for (int e = threadIdx.x; e < n_rows; e += blockDim.x)
      z[e] = logits[(size_t)t * n_rows + e] + (add_bias && e < n_experts ? bias[e] : 0.f);
  } else {
    const T* row = h + (size_t)t * width;
    const bool vec = width % 4 == 0 && ((uintptr_t)w % 16 == 0) && ((uintptr_t)h % 16 == 0);
    for (int e = warp; e < n_rows; e += 16) {
      const float* we = w + (size_t)e * width;
      float s[4] = {0.f, 0.f, 0.f, 0.f};  // four partial sums a lane
      if (vec) {
        // 16 bytes of the weight row and four activations a lane and trip, eight trips' loads in flight together
#pragma unroll 8
        for (int i = lane * 4; i < width; i += 128) {
          const float4 wv = *reinterpret_cast<const float4*>(we + i);
          float hv[4];
          if constexpr (sizeof(T) == 4) {
            const float4 x = *reinterpret_cast<const float4*>(row + i);
            hv[0] = x.x; hv[1] = x.y; hv[2] = x.z; hv[3] = x.w;
          } else {
            const uint2 x = *reinterpret_cast<const uint2*>(row + i);
            const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&x.x));
            const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&x.y));
            hv[0] = lo.x; hv[1] = lo.y; hv[2] = hi.x; hv[3] = hi.y;
          }
          s[0] = fmaf(hv[0], wv.x, s[0]);
          s[1] = fmaf(hv[1], wv.y, s[1]);
          s[2] = fmaf(hv[2], wv.z, s[2]);
          s[3] = fmaf(hv[3], wv.w, s[3]);
        }
      } else {
        for (int i = lane; i < width; i += 32) s[0] = fmaf(to_float(row[i]), we[i], s[0]);
      }
      const float total = warp_sum((s[0] + s[1]) + (s[2] + s[3]));
      if (lane == 0) z[e] = total + (add_bias && e < n_experts ? bias[e] : 0.f);
    }
  }
  __syncthreads();
  if (warp != 0) return;
  if (form.gate_out && lane == 0) form.gate_out[t] = 1.f / (1.f + expf(-z[n_experts]));
  if (form.all_scores) {
    // scores over every expert; the choice goes by score + correction (or by score inside the kept groups), the
    // weights by the scores alone:  weight_j = score_j / (sum of the chosen scores + 1e-20) * scale
    float* choice = z + n_rows;  // [n_experts]
    if (form.all_scores == 2) {
      float* group_score = choice + n_experts;  // [groups]
      const int per = n_experts / form.groups;
      for (int e = lane; e < n_experts; e += 32) z[e] = 1.f / (1.f + expf(-z[e]));
      __syncwarp();
      for (int g = lane; g < form.groups; g += 32) {
        float a = -INFINITY, b = -INFINITY;  // the run's top two scores
        for (int e = g * per; e < (g + 1) * per; ++e) {
          const float v = z[e];
          if (v > a) { b = a; a = v; } else if (v > b) { b = v; }
        }
        group_score[g] = per > 1 ? a + b : a;
      }
      for (int e = lane; e < n_experts; e += 32) choice[e] = -INFINITY;
      __syncwarp();
      for (int j = 0; j < form.groups_kept; ++j) {
        float best = -INFINITY;
        int at = 0x7fffffff;
        for (int g = lane; g < form.groups; g += 32) {
          const float v = group_score[g];
          if (v > best || (v == best && g < at)) { best = v; at = g; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
          const float ob = __shfl_xor_sync(0xffffffffu, best, o);
          const int oa = __shfl_xor_sync(0xffffffffu, at, o);
          if (ob > best || (ob == best && oa < at)) { best = ob; at = oa; }
        }
        if (at >= form.groups) break;  // nothing comparable was left
        for (int e = at * per + lane; e < (at + 1) * per; e += 32) choice[e] = z[e];
        if (lane == 0) group_score[at] = -INFINITY;
        __syncwarp();
      }
    } else {
    float top_z = -INFINITY;
    for (int e = lane; e < n_experts; e += 32) top_z = fmaxf(top_z, z[e]);
    top_z = warp_max(top_z);
    float denom = 0.f;
    for (int e = lane; e < n_experts; e += 32) denom += expf(z[e] - top_z);
    denom = warp_sum(denom);
    for (int e = lane; e < n_experts; e += 32) {
      const float sc = expf(z[e] - top_z) / denom;
      z[e] = sc;
      choice[e] = sc + (bias ? bias[e] : 0.f);
    }
    }
    __syncwarp();
    float chosen_sum = 0.f;
    for (int j = 0; j < top; ++j) {
      float best = -INFINITY;
      int at = 0x7fffffff;
      for (int e = lane; e < n_experts; e += 32) {
        const float v = choice[e];
        if (v > best || (v == best && e < at)) { best = v; at = e; }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int oa = __shfl_xor_sync(0xffffffffu, at, o);
        if (ob > best || (ob == best && oa < at)) { best = ob; at = oa; }
      }
      if (at >= n_experts) at = j;
      const float sc = z[at];
      chosen_sum += sc;
      if (lane == 0) {
        chosen[(size_t)t * top + j] = at;
        weight[(size_t)t * top + j] = sc;
        choice[at] = -INFINITY;
      }
      __syncwarp();
    }
    if (lane < top) weight[(size_t)t * top + lane] = weight[(size_t)t * top + lane] / (chosen_sum + 1e-20f) * form.scale;
    return;
  }
  float first = 0.f, total = 0.f;
  for (int j = 0; j < top; ++j) {
    float best = -INFINITY;
    int at = 0x7fffffff;
    for (int e = lane; e < n_experts; e += 32) {
      const float v = z[e];
      if (v > best || (v == best && e < at)) { best = v; at = e; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oa = __shfl_xor_sync(0xffffffffu, at, o);
      if (ob > best || (ob == best && oa < at)) { best = ob; at = oa; }
    }
    if (at >= n_experts) at = j;  // nothing comparable was left (not-a-number logits): any expert that exists
    if (j == 0) first = best;
    const float p = expf(best - first);
    total += p;
    if (lane == 0) {
      chosen[(size_t)t * top + j] = at;
      weight[(size_t)t * top + j] = p;
      z[at] = -INFINITY;
    }
    __syncwarp();
  }
  if (lane < top) weight[(size_t)t * top + lane] /= total;
}

// ---- sort ----------------------------------------------------------------------------------------------------- //
__global__ void __launch_bounds__(1024) moe_sort_kernel(const int* __restrict__ chosen, MoePlan plan, int n_pairs,
                                                        int n_experts, int bm, int n_real) {
  extern __shared__ int sort_smem[];
  int* counts = sort_smem;                 // [E]
  int* offsets = counts + n_experts;       // [E + 1]
  int* tile_off = offsets + n_experts + 1; // [E + 1]
  int* cursor = tile_off + n_experts + 1;  // [E]
  for (int e = threadIdx.x; e < n_experts; e += blockDim.x) counts[e] = 0;
  __syncthreads();
  for (int p = threadIdx.x; p < n_pairs; p += blockDim.x) atomicAdd(&counts[chosen[p]], 1);
  __syncthreads();
  if (threadIdx.x == 0) {
    offsets[0] = 0;
    tile_off[0] = 0;
    for (int e = 0; e < n_experts; ++e) {
      offsets[e + 1] = offsets[e] + counts[e];
      // experts past n_real have no matrices (they hand their input on): places, but no tiles
      tile_off[e + 1] = tile_off[e] + (e < n_real ? (counts[e] + bm - 1) / bm : 0);
    }
    plan.n_tiles[0] = tile_off[n_experts];
  }
  __syncthreads();
  for (int e = threadIdx.x; e <= n_experts; e += blockDim.x) plan.offsets[e] = offsets[e];
  for (int e = threadIdx.x; e < n_experts; e += blockDim.x) {
    cursor[e] = offsets[e];
    for (int i = tile_off[e]; i < tile_off[e + 1]; ++i) {
      plan.tile_expert[i] = e;
      plan.tile_row0[i] = offsets[e] + (i - tile_off[e]) * bm;
    }
  }
  __syncthreads();
  // a pair's place among its expert's rows depends on the order of arrival; no result depends on the place
  for (int p = threadIdx.x; p < n_pairs; p += blockDim.x) plan.order[atomicAdd(&cursor[chosen[p]], 1)] = p;
}

// ---- the plain products --------------------------------------------------------------------------------------- //
constexpr int SIMT_BK = 128;

template <typename T>
__device__ __forceinline__ void load_chunk(const T* p, int n, bool vec, float* out) {
  // n <= 16 / sizeof(T) consecutive elements as floats
  constexpr int PAD = 16 / sizeof(T);
  if (vec && n == PAD) {
    if constexpr (sizeof(T) == 4) {
      const float4 v = *reinterpret_cast<const float4*>(p);
      out[0] = v.x; out[1] = v.y; out[2] = v.z; out[3] = v.w;
    } else {
      const uint4 v = *reinterpret_cast<const uint4*>(p);
      const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 f = __bfloat1622float2(h2[i]);
        out[2 * i] = f.x;
        out[2 * i + 1] = f.y;
      }
    }
  } else {
    for (int i = 0; i < PAD; ++i) out[i] = i < n ? to_float(p[i]) : 0.f;
  }
}

__device__ __forceinline__ float gelu_erf_f(float z) { return 0.5f * z * (1.f + erff(z * 0.70710678118654752f)); }

// KIND 1: A rows are the tokens of the tile's pairs, two accumulators per row (gate, up), out act[place, n] =
// silu(gate) * up.  KIND 2: the same rows, one accumulator, out act[place, n] = gelu(up) (erf form).
// KIND 0: A rows are act[place], out y[pair, n] = weight[pair] * sum, float32.
template <typename T, int KIND>
__global__ void __launch_bounds__(128) moe_simt_kernel(MoeProductArgs a) {
  constexpr bool GATE_UP = KIND == 1;
  constexpr bool GATHER = KIND != 0;
  const int tile = blockIdx.x;
  if (tile >= a.plan.n_tiles[0]) return;
  constexpr int PAD = 16 / sizeof(T);
  __shared__ float a_s[MOE_SIMT_BM][SIMT_BK + 1];
  __shared__ int row_src[MOE_SIMT_BM];
  const int e = a.plan.tile_expert[tile], row0 = a.plan.tile_row0[tile];
  const int rows = min(MOE_SIMT_BM, a.plan.offsets[e + 1] - row0);
  const int tid = threadIdx.x;
  const int col = blockIdx.y * 128 + tid;
  const int K = a.k, N = a.n;
  if (tid < MOE_SIMT_BM) {
    int src = -1;
    if (tid < rows) src = GATHER ? a.plan.order[row0 + tid] / a.top : row0 + tid;
    row_src[tid] = src;
  }
  __syncthreads();
  const T* w0 = (const T*)a.w + ((size_t)e * (GATE_UP ? 2 * N : N) + min(col, N - 1)) * K;
  const T* w1 = w0 + (size_t)N * K;  // the up row (GATE_UP only)
  const bool vec = K % PAD == 0 && ((uintptr_t)a.w % 16 == 0);
  float acc0[MOE_SIMT_BM], acc1[GATE_UP ? MOE_SIMT_BM : 1];
#pragma unroll
  for (int r = 0; r < MOE_SIMT_BM; ++r) acc0[r] = 0.f;
#pragma unroll
  for (int r = 0; r < (GATE_UP ? MOE_SIMT_BM : 1); ++r) acc1[r] = 0.f;
  for (int k0 = 0; k0 < K; k0 += SIMT_BK) {
    const int kn = min(SIMT_BK, K - k0);
    for (int idx = tid; idx < MOE_SIMT_BM * SIMT_BK; idx += 128) {
      const int r = idx / SIMT_BK, c = idx % SIMT_BK;
      const int src = row_src[r];
      a_s[r][c] = (src >= 0 && c < kn) ? to_float(((const T*)a.a)[(size_t)src * K + k0 + c]) : 0.f;
    }
    __syncthreads();
    for (int c = 0; c < kn; c += PAD) {
      float wv0[PAD], wv1[PAD];
      load_chunk<T>(w0 + k0 + c, min(PAD, kn - c), vec, wv0);
      if (GATE_UP) load_chunk<T>(w1 + k0 + c, min(PAD, kn - c), vec, wv1);
#pragma unroll
      for (int u = 0; u < PAD; ++u) {
#pragma unroll
        for (int r = 0; r < MOE_SIMT_BM; ++r) {
          const float av = a_s[r][c + u];  // columns past kn hold zeros
          acc0[r] = fmaf(av, wv0[u], acc0[r]);
          if (GATE_UP) acc1[r] = fmaf(av, wv1[u], acc1[r]);
        }
      }
    }
    __syncthreads();
  }
  if (col >= N) return;
#pragma unroll
  for (int r = 0; r < MOE_SIMT_BM; ++r) {
    if (r >= rows) break;
    if (GATE_UP) {
      const float g = acc0[r];
      ((T*)a.out)[(size_t)(row0 + r) * N + col] = from_float<T>(g / (1.f + expf(-g)) * acc1[r]);
    } else if (KIND == 2) {
      ((T*)a.out)[(size_t)(row0 + r) * N + col] = from_float<T>(gelu_erf_f(acc0[r]));
    } else {
      const int pair = a.plan.order[row0 + r];
      ((float*)a.out)[(size_t)pair * N + col] = a.pair_weight[pair] * acc0[r];
    }
  }
}

// ---- combine -------------------------------------------------------------------------------------------------- //
// Experts past n_real have no matrices: their share is weight * the token's own row h.  other_gate: a factor per
// token on the other part's output.
struct CombineExtras {
  const int* chosen;          // [tokens, top] or null: every choice has a row in y
  const float* pair_weight;   // [tokens, top]
  const void* h;              // [tokens, width] of the output's dtype
  int n_real;
  const float* other_gate;    // [tokens] or null
};

template <typename T>
__global__ void moe_combine_kernel(const float* __restrict__ y, const T* __restrict__ other, T* __restrict__ out,
                                   size_t total, int width, int top, CombineExtras x) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const size_t t = i / width;
    const int c = (int)(i % width);
    float s = 0.f;
    for (int j = 0; j < top; ++j) {
      if (x.chosen && x.chosen[t * top + j] >= x.n_real)
        s += x.pair_weight[t * top + j] * to_float(((const T*)x.h)[i]);
      else
        s += y[(t * top + j) * width + c];
    }
    if (other) s += (x.other_gate ? x.other_gate[t] : 1.f) * to_float(other[i]);
    out[i] = from_float<T>(s);
  }
}

}  // namespace mll

MLL_API int mll_moe_simt_rows() { return MOE_SIMT_BM; }

// h: [n_tokens, width] of `dtype`; w: float32 [n_experts (+ 1 with gate_out), width]; bias: float32 [n_experts] or null;
// logits: null, or float32 [n_tokens, n_experts (+ 1)] = h w^T formed by the caller (h and w are then not read);
// all_scores, scale, gate_out: see RouteForm;
// chosen: int32 [n_tokens, top]; weight: float32 [n_tokens, top].
MLL_API int mll_moe_route(const void* h, const float* w, const float* bias, const float* logits, int* chosen,
                          float* weight, int dtype, int n_tokens, int width, int n_experts, int top, int all_scores,
                          float scale, float* gate_out, int groups, int groups_kept, cudaStream_t stream) {
  MLL_REQUIRE(n_tokens >= 0 && width > 0 && n_experts > 0 && top > 0 && top <= n_experts && top <= 32,
              "moe route: bad sizes tokens=%d width=%d experts=%d top=%d", n_tokens, width, n_experts, top);
  MLL_REQUIRE(n_experts <= 2048, "moe route: %d experts (at most 2048)", n_experts);
  if (n_tokens == 0) return 0;
  MLL_REQUIRE(all_scores >= 0 && all_scores <= 2, "moe route: unknown scoring %d", all_scores);
  if (all_scores == 2) {
    MLL_REQUIRE(groups >= 1 && n_experts % groups == 0 && groups_kept >= 1 && groups_kept <= groups,
                "moe route: %d experts in %d groups of which %d are kept", n_experts, groups, groups_kept);
    MLL_REQUIRE(top <= groups_kept * (n_experts / groups), "moe route: top %d of %d experts in the kept groups", top,
                groups_kept * (n_experts / groups));
  } else {
    groups = groups_kept = 0;
  }
  const size_t smem = (size_t)(2 * n_experts + 1 + groups) * sizeof(float);
  const mll::RouteForm form{all_scores, scale, gate_out, groups, groups_kept};
  if (dtype == MLL_F32)
    MLL_LAUNCH((mll::moe_route_kernel<float>), n_tokens, 512, smem, stream, (const float*)h, w, bias, logits, chosen,
               weight, n_tokens, width, n_experts, top, form);
  else if (dtype == MLL_BF16)
    MLL_LAUNCH((mll::moe_route_kernel<__nv_bfloat16>), n_tokens, 512, smem, stream, (const __nv_bfloat16*)h, w, bias,
               logits, chosen, weight, n_tokens, width, n_experts, top, form);
  else
    MLL_REQUIRE(false, "moe route: unknown dtype %d", dtype);
  MLL_LAUNCH_CHECK();
  return 0;
}

// chosen: int32 [n_pairs]; order: int32 [n_pairs]; offsets: int32 [n_experts + 1]; tile_expert, tile_row0: int32
// [n_pairs / bm + n_experts]; n_tiles: int32 [1].
MLL_API int mll_moe_sort(const int* chosen, int* order, int* offsets, int* tile_expert, int* tile_row0, int* n_tiles,
                         int n_pairs, int n_experts, int bm, int n_real, cudaStream_t stream) {
  MLL_REQUIRE(n_pairs >= 0 && n_experts > 0 && n_experts <= 2048 && bm > 0, "moe sort: bad sizes");
  MLL_REQUIRE(n_real >= 0 && n_real <= n_experts, "moe sort: %d of %d experts have matrices", n_real, n_experts);
  if (n_pairs == 0) return 0;
  const size_t smem = (size_t)(4 * n_experts + 2) * sizeof(int);
  MLL_LAUNCH((mll::moe_sort_kernel), 1, 1024, smem, stream, chosen,
             mll::MoePlan{order, offsets, tile_expert, tile_row0, n_tiles}, n_pairs, n_experts, bm, n_real);
  MLL_LAUNCH_CHECK();
  return 0;
}

static int moe_check(const char* what, int max_tiles, int k, int n, int top) {
  MLL_REQUIRE(max_tiles > 0 && k > 0 && n > 0 && top > 0, "%s: bad sizes tiles=%d k=%d n=%d top=%d", what, max_tiles, k, n, top);
  MLL_REQUIRE((n + 127) / 128 <= 65535, "%s: %d columns are too many for one launch", what, n);
  return 0;
}

// act[place, :] = silu(W_gate,e h[token]) * (W_up,e h[token]) for every place of the sorted pairs (form 0), or
// gelu(W_up,e h[token]) in the erf form (form 1).
// h: [n_tokens, width]; w: [n_experts, 2 inter, width] (an expert's gate rows, then its up rows; form 1: [n_experts,
// inter, width]); act: [n_pairs, inter].
MLL_API int mll_moe_gate_up(const void* h, const void* w, void* act, const int* order, const int* offsets,
                            const int* tile_expert, const int* tile_row0, const int* n_tiles, int dtype, int max_tiles,
                            int width, int inter, int top, int form, cudaStream_t stream) {
  if (moe_check("moe gate_up", max_tiles, width, inter, top)) return -1;
  MLL_REQUIRE(form == 0 || form == 1, "moe gate_up: unknown expert form %d", form);
  mll::MoeProductArgs a{h, w, act, nullptr, mll::MoePlan{(int*)order, (int*)offsets, (int*)tile_expert, (int*)tile_row0,
                                                         (int*)n_tiles}, width, inter, top};
  const dim3 grid(max_tiles, (inter + 127) / 128);
  if (dtype == MLL_F32 && form == 0)
    MLL_LAUNCH((mll::moe_simt_kernel<float, 1>), grid, 128, 0, stream, a);
  else if (dtype == MLL_F32)
    MLL_LAUNCH((mll::moe_simt_kernel<float, 2>), grid, 128, 0, stream, a);
  else if (dtype == MLL_BF16 && form == 0)
    MLL_LAUNCH((mll::moe_simt_kernel<__nv_bfloat16, 1>), grid, 128, 0, stream, a);
  else if (dtype == MLL_BF16)
    MLL_LAUNCH((mll::moe_simt_kernel<__nv_bfloat16, 2>), grid, 128, 0, stream, a);
  else
    MLL_REQUIRE(false, "moe gate_up: unknown dtype %d", dtype);
  MLL_LAUNCH_CHECK();
  return 0;
}

// y[pair, :] = weight[pair] * W_down,e act[place] (float32).  act: [n_pairs, inter]; w: [n_experts, width, inter].
MLL_API int mll_moe_down(const void* act, const void* w, float* y, const float* pair_weight, const int* order,
                         const int* offsets, const int* tile_expert, const int* tile_row0, const int* n_tiles, int dtype,
                         int max_tiles, int inter, int width, int top, cudaStream_t stream) {
  if (moe_check("moe down", max_tiles, inter, width, top)) return -1;
  mll::MoeProductArgs a{act, w, y, pair_weight, mll::MoePlan{(int*)order, (int*)offsets, (int*)tile_expert,
                                                             (int*)tile_row0, (int*)n_tiles}, inter, width, top};
  const dim3 grid(max_tiles, (width + 127) / 128);
  if (dtype == MLL_F32)
    MLL_LAUNCH((mll::moe_simt_kernel<float, 0>), grid, 128, 0, stream, a);
  else if (dtype == MLL_BF16)
    MLL_LAUNCH((mll::moe_simt_kernel<__nv_bfloat16, 0>), grid, 128, 0, stream, a);
  else
    MLL_REQUIRE(false, "moe down: unknown dtype %d", dtype);
  MLL_LAUNCH_CHECK();
  return 0;
}

// out[t, :] = y[t * top, :] + ... + y[t * top + top - 1, :] (+ other[t, :]); y float32, other and out of `dtype`.
// chosen (with pair_weight, h, n_real): choices of experts past n_real add pair_weight * h[t] instead of a row of y.
// other_gate: float32 [n_tokens], a factor on `other`.
MLL_API int mll_moe_combine(const float* y, const void* other, void* out, int dtype, int n_tokens, int width, int top,
                            const int* chosen, const float* pair_weight, const void* h, int n_real,
                            const float* other_gate, cudaStream_t stream) {
  MLL_REQUIRE(n_tokens >= 0 && width > 0 && top > 0, "moe combine: bad sizes");
  MLL_REQUIRE(!chosen || (pair_weight && h), "moe combine: pass-through experts need the weights and the input rows");
  const mll::CombineExtras extras{chosen, pair_weight, h, n_real, other_gate};
  if (n_tokens == 0) return 0;
  const size_t total = (size_t)n_tokens * width;
  long long blocks = (long long)((total + 255) / 256);
  if (blocks > mll_sm_count() * 16) blocks = mll_sm_count() * 16;
  if (dtype == MLL_F32)
    MLL_LAUNCH((mll::moe_combine_kernel<float>), (int)blocks, 256, 0, stream, y, (const float*)other, (float*)out, total,
               width, top, extras);
  else if (dtype == MLL_BF16)
    MLL_LAUNCH((mll::moe_combine_kernel<__nv_bfloat16>), (int)blocks, 256, 0, stream, y, (const __nv_bfloat16*)other,
               (__nv_bfloat16*)out, total, width, top, extras);
  else
    MLL_REQUIRE(false, "moe combine: unknown dtype %d", dtype);
  MLL_LAUNCH_CHECK();
  return 0;
}
