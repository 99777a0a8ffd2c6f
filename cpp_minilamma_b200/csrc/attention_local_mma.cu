// Prompt steps of the chunked attention (attention_local.cu) on tensor cores, bfloat16: the flash-style
// mma.sync kernel of attention_mma_prefill.cu with head sizes of their own for keys (d) and values (dv),
// an explicit scale, and the chunk mask (key j visible from query i iff j <= i and j / chunk == i / chunk).
// The kernel is instantiated for padded sizes DK, DV in {32, 64, 128, 256}; the real d and dv (multiples of
// 8, so that rows are whole 16-byte words) are runtime values and the padding columns are zero-filled in
// shared memory.  A tile starts at the first page that its first row's chunk (or window) reaches.  With a window that
// keeps the sequence's first tokens (`keep_first`) the pages of those tokens are walked first, then the window's; a
// capped score is cap * tanh(scale * s / cap).
//
// The same kernel serves steps of single tokens (`heads_as_rows`): a block then takes one sequence and one kv head,
// and its rows are the query heads of that kv head's group (up to 64 a block), all at the sequence's last
// position - few rows of a 16-row tensor-core tile when the group is small, a full tile when many heads share one
// key/value head (attention over a latent).  The context may be cut into n_splits runs of pages, a block each
// (grid z): the blocks then leave their unnormalised results with their maxima and sums in scratch memory and a
// second kernel merges them in split order; a sink is counted by the split that holds the first keys.
#include "attention_decode.cuh"
#include "common.cuh"

namespace mll {

struct LocalMmaArgs {
  const __nv_bfloat16* q;        // [T, Hq * d]
  const __nv_bfloat16* k_cache;  // [n_pages, Hk, PAGE, d]
  const __nv_bfloat16* v_cache;  // [n_pages, Hk, PAGE, dv]
  const int* seq_slot;
  const int* seq_ctx;
  const int* seq_qstart;
  const int* seq_qlen;
  const int* tile_seq;
  const int* tile_row0;
  const int* block_table;
  __nv_bfloat16* out;            // [T, Hq * dv]
  int n_heads, n_kv_heads, max_blocks, window, chunk, d, dv;
  float scale_log2;
  int sink;                      // 1: one more term exp(sink value) in the softmax's denominator, without a value
  const float* sink_values;      // [Hq] the sink's score per query head (natural units, unscaled), or null: 0
  int heads_as_rows;             // 1: single tokens; grid (sequences, kv heads * chunks of 64 heads of a group)
  int v_ld;                      // elements between value rows: dv, or d when the values are the keys' leading columns
  int n_splits;                  // heads_as_rows only: blocks per (sequence, kv head, head chunk) along the context
  float* part_o;                 // [sequences, heads, n_splits, dv] unnormalised results (n_splits > 1)
  float* part_ml;                // [sequences, heads, n_splits, 2] maximum (log2 units) and sum
  int keep_first;                // with a window: keys at positions below this stay visible
  float softcap;                 // > 0: score <- softcap * tanh(score / softcap), in natural units
  float scale;                   // the scale in natural units (scale_log2 = scale * log2 e)
};

// tanh(x) = 1 - 2 / (1 + e^(2x)) on the fast exponential and division: absolute error near 1e-6, which a capped score
// (cap * tanh) of a bfloat16 run does not see; large |x| saturates to +-1 (e^(2x) overflows to infinity or falls to 0).
__device__ __forceinline__ float fast_tanh(float x) { return 1.f - __fdividef(2.f, 1.f + __expf(2.f * x)); }

template <int DK, int DV>
struct LocalMmaSmem {
  static constexpr int KS = DK + 8, VS = DV + 8;
  static constexpr int KTILE = 64 * KS, VTILE = 64 * VS;
  static constexpr size_t BYTES = (size_t)2 * (KTILE + VTILE) * 2;
};

template <int DK, int DV>
__global__ void __launch_bounds__(128) local_prefill_mma_kernel(LocalMmaArgs a) {
  using L = LocalMmaSmem<DK, DV>;
  constexpr int KSTEPS = DK / 16;
  constexpr int NT_OUT = DV / 8;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  // Values that are the keys' leading columns are read from the key tile itself: a page is loaded once and a stage
  // is half the size (three blocks a multiprocessor instead of one at keys of 256).
  const bool v_in_k = a.v_cache == a.k_cache;
  const int stage_elems = v_in_k ? L::KTILE : L::KTILE + L::VTILE;
  const int vs = v_in_k ? L::KS : L::VS;                             // elements between value rows in shared memory
  __nv_bfloat16* kv_s = reinterpret_cast<__nv_bfloat16*>(smem_raw);  // [2 stages][K 64 x KS (, V 64 x VS)]
  __nv_bfloat16* q_s = kv_s + stage_elems;                           // the query tile passes through stage 1's K tile

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int group = a.n_heads / a.n_kv_heads;
  const bool by_heads = a.heads_as_rows != 0;
  const int head_chunks = (group + 63) / 64;
  const int seq = by_heads ? blockIdx.x : a.tile_seq[blockIdx.x], row0 = by_heads ? 0 : a.tile_row0[blockIdx.x];
  const int kvh = by_heads ? blockIdx.y / head_chunks : blockIdx.y / group;
  const int h = by_heads ? kvh * group + (blockIdx.y % head_chunks) * 64 : blockIdx.y;  // the (first) head of the block
  const int ctx = a.seq_ctx[seq], qlen = by_heads ? 1 : a.seq_qlen[seq];
  const int rows = by_heads ? min(64, kvh * group + group - h) : min(64, qlen - row0);
  const int pos0 = ctx - qlen + row0;
  const int pos_step = by_heads ? 0 : 1;  // rows are consecutive positions, or heads at one position
  const int d = a.d, dv = a.dv;
  const size_t q_stride = by_heads ? d : (size_t)a.n_heads * d, o_stride = by_heads ? dv : (size_t)a.n_heads * dv;
  const int* table = a.block_table + (size_t)a.seq_slot[seq] * a.max_blocks;
  constexpr int KCPR = DK / 8, VCPR = DV / 8;  // 16-byte words per padded row

  {
    const __nv_bfloat16* qg = a.q + ((size_t)a.seq_qstart[seq] + row0) * a.n_heads * d + (size_t)h * d;
    for (int c = tid; c < 64 * KCPR; c += 128) {
      const int r = c / KCPR, cc = c % KCPR;
      const bool in = r < rows && cc * 8 < d;
      cp_async16_zfill(q_s + r * L::KS + cc * 8, qg + (size_t)min(r, rows - 1) * q_stride + (in ? cc * 8 : 0), in);
    }
  }
  auto load_page = [&](int page_index, int stage) {
    const int page = table[page_index];
    const __nv_bfloat16* kg = a.k_cache + ((size_t)page * a.n_kv_heads + kvh) * MLL_PAGE * d;
    const __nv_bfloat16* vg = a.v_cache + ((size_t)page * a.n_kv_heads + kvh) * MLL_PAGE * a.v_ld;
    __nv_bfloat16* kd = kv_s + (size_t)stage * stage_elems;
    __nv_bfloat16* vd = kd + L::KTILE;
    const int valid_rows = ctx - page_index * MLL_PAGE;  // rows past the cached length hold no data
    for (int c = tid; c < MLL_PAGE * KCPR; c += 128) {
      const int r = c / KCPR, cc = c % KCPR;
      const bool in = cc * 8 < d && r < valid_rows;
      cp_async16_zfill(kd + r * L::KS + cc * 8, kg + (size_t)r * d + (in ? cc * 8 : 0), in);
    }
    for (int c = tid; c < (v_in_k ? 0 : MLL_PAGE * VCPR); c += 128) {
      const int r = c / VCPR, cc = c % VCPR;
      const bool in = cc * 8 < dv && r < valid_rows;
      cp_async16_zfill(vd + r * L::VS + cc * 8, vg + (size_t)r * a.v_ld + (in ? cc * 8 : 0), in);
    }
  };

  int first_key = a.chunk > 0 ? (pos0 / a.chunk) * a.chunk : 0;  // of the tile's first row; later rows reach no further back
  if (a.window > 0) first_key = max(first_key, pos0 - a.window + 1);
  const int last_pos = pos0 + (rows - 1) * pos_step;
  const int last_chunk_start = a.chunk > 0 ? (last_pos / a.chunk) * a.chunk : 0;
  const int p_first = first_key / MLL_PAGE, p_last = last_pos / MLL_PAGE;
  // kept first tokens in front of the window: their pages are walked before the window's.  The walk's index w stands
  // for page w below n_kept and for page p_first + (w - n_kept) from there on.
  const int kept = (a.window > 0 && a.keep_first > 0) ? min(a.keep_first, first_key) : 0;
  const int n_kept = min((kept + MLL_PAGE - 1) / MLL_PAGE, p_first);
  auto page_at = [&](int w) { return w < n_kept ? w : p_first + (w - n_kept); };
  const int w_last = n_kept + (p_last - p_first);
  int pb = 0, pe = w_last;  // this block's run of the walk
  if (a.n_splits > 1) {
    const int per = (w_last + a.n_splits) / a.n_splits;
    pb = (int)blockIdx.z * per;
    pe = min(w_last, pb + per - 1);
  }
  if (pb <= pe) load_page(page_at(pb), 0);
  cp_async_commit();

  unsigned qf[KSTEPS][4];
  float o[NT_OUT][4];
#pragma unroll
  for (int n = 0; n < NT_OUT; ++n)
#pragma unroll
    for (int i = 0; i < 4; ++i) o[n][i] = 0.f;
  // with a sink every row starts as if it had seen one key that scores 0 and has no value
  const bool sink = a.sink && (a.n_splits <= 1 || blockIdx.z == 0);
  float m_run[2] = {sink ? 0.f : -INFINITY, sink ? 0.f : -INFINITY}, l_run[2] = {sink ? 1.f : 0.f, sink ? 1.f : 0.f};
  if (sink && a.sink_values) {  // a learned sink: the row starts at the sink's score (log2 units, like the scores)
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const int row = warp * 16 + g + 8 * r;
      m_run[r] = a.sink_values[by_heads ? h + min(row, rows - 1) : h] * 1.4426950408889634f;
    }
  }

  const float cap_log2 = a.softcap * 1.4426950408889634f, scale_over_cap = a.softcap > 0.f ? a.scale / a.softcap : 0.f;
  // single tokens: a warp whose 16 rows lie past the group's heads has nothing to compute; it still loads and waits
  const bool idle = by_heads && warp * 16 >= rows;
  for (int w = pb; w <= pe; ++w) {
    const int p = page_at(w);
    const int stage = (w - pb) & 1;
    cp_async_wait<0>();
    __syncthreads();
    if (w == pb) {
#pragma unroll
      for (int ks = 0; ks < KSTEPS; ++ks)
        ldmatrix_x4(qf[ks], q_s + (warp * 16 + (lane & 7) + (((lane >> 3) & 1) << 3)) * L::KS + ks * 16 +
                                ((lane >> 4) << 3));
      __syncthreads();
    }
    if (w < pe) load_page(page_at(w + 1), stage ^ 1);
    cp_async_commit();
    const __nv_bfloat16* kt = kv_s + (size_t)stage * stage_elems;
    const __nv_bfloat16* vt = v_in_k ? kt : kt + L::KTILE;
    if (idle) continue;

    float s_acc[8][4];
#pragma unroll
    for (int n = 0; n < 8; ++n)
#pragma unroll
      for (int i = 0; i < 4; ++i) s_acc[n][i] = 0.f;
#pragma unroll
    for (int ks = 0; ks < KSTEPS; ++ks) {
#pragma unroll
      for (int n = 0; n < 8; n += 2) {
        unsigned kb[4];
        const int key = n * 8 + (lane & 7) + ((lane >> 4) << 3);
        const int dim = ks * 16 + (((lane >> 3) & 1) << 3);
        ldmatrix_x4(kb, kt + key * L::KS + dim);
        mma_16816(s_acc[n], qf[ks], kb[0], kb[1]);
        mma_16816(s_acc[n + 1], qf[ks], kb[2], kb[3]);
      }
    }
    // mask where the page meets the diagonal, a chunk's or the window's edge, or the tile's end
    // ... or the window's far edge: keys at or below the last row's edge that are not all kept first tokens
    const bool window_edge = a.window > 0 && p * MLL_PAGE <= last_pos - a.window && p * MLL_PAGE + MLL_PAGE - 1 >= a.keep_first;
    const bool needs_mask = (p * MLL_PAGE + MLL_PAGE - 1 > pos0 + warp * 16 * pos_step) || window_edge || rows < 64 ||
                            p * MLL_PAGE < last_chunk_start;
#pragma unroll
    for (int n = 0; n < 8; ++n)
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        float v = a.softcap > 0.f ? cap_log2 * fast_tanh(s_acc[n][i] * scale_over_cap) : s_acc[n][i] * a.scale_log2;
        if (needs_mask) {
          const int row = warp * 16 + g + ((i >> 1) << 3);
          const int qpos = pos0 + row * pos_step;
          const int kpos = p * MLL_PAGE + n * 8 + 2 * t + (i & 1);
          const bool ok = row < rows && kpos <= qpos && (a.window <= 0 || kpos > qpos - a.window || kpos < a.keep_first) &&
                          (a.chunk <= 0 || kpos >= (qpos / a.chunk) * a.chunk);
          v = ok ? v : -INFINITY;
        }
        s_acc[n][i] = v;
      }
    float alpha[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      float mx = -INFINITY;
#pragma unroll
      for (int n = 0; n < 8; ++n) mx = fmaxf(mx, fmaxf(s_acc[n][2 * r], s_acc[n][2 * r + 1]));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
      const float m_new = fmaxf(m_run[r], mx);
      const float base = m_new > -INFINITY ? m_new : 0.f;  // a row with nothing visible yet stays at zero weight
      alpha[r] = exp2f(m_run[r] - base);
      float sum = 0.f;
#pragma unroll
      for (int n = 0; n < 8; ++n) {
        const float p0 = exp2f(s_acc[n][2 * r] - base), p1 = exp2f(s_acc[n][2 * r + 1] - base);
        s_acc[n][2 * r] = p0;
        s_acc[n][2 * r + 1] = p1;
        sum += p0 + p1;
      }
      sum += __shfl_xor_sync(0xffffffffu, sum, 1);
      sum += __shfl_xor_sync(0xffffffffu, sum, 2);
      l_run[r] = l_run[r] * alpha[r] + sum;
      m_run[r] = m_new;
    }
#pragma unroll
    for (int n = 0; n < NT_OUT; ++n) {
      o[n][0] *= alpha[0];
      o[n][1] *= alpha[0];
      o[n][2] *= alpha[1];
      o[n][3] *= alpha[1];
    }
#pragma unroll
    for (int ks = 0; ks < 4; ++ks) {
      unsigned pa[4];
      pa[0] = pack_bf162(s_acc[2 * ks][0], s_acc[2 * ks][1]);
      pa[1] = pack_bf162(s_acc[2 * ks][2], s_acc[2 * ks][3]);
      pa[2] = pack_bf162(s_acc[2 * ks + 1][0], s_acc[2 * ks + 1][1]);
      pa[3] = pack_bf162(s_acc[2 * ks + 1][2], s_acc[2 * ks + 1][3]);
#pragma unroll
      for (int n = 0; n < NT_OUT; n += 2) {
        unsigned vb[4];
        const int key = ks * 16 + (lane & 7) + (((lane >> 3) & 1) << 3);
        const int col = (n + (lane >> 4)) * 8;
        ldmatrix_x4_trans(vb, vt + key * vs + col);
        mma_16816(o[n], pa, vb[0], vb[1]);
        mma_16816(o[n + 1], pa, vb[2], vb[3]);
      }
    }
  }
  cp_async_wait<0>();

#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int row = warp * 16 + g + 8 * r;
    if (row >= rows) continue;
    if (a.n_splits > 1) {
      const size_t at = (((size_t)seq * a.n_heads + h + row) * a.n_splits + blockIdx.z);
#pragma unroll
      for (int n = 0; n < NT_OUT; ++n)
        if (n * 8 + 2 * t < dv)
          *reinterpret_cast<float2*>(a.part_o + at * dv + n * 8 + 2 * t) = make_float2(o[n][2 * r], o[n][2 * r + 1]);
      if (t == 0) {
        a.part_ml[at * 2] = m_run[r];
        a.part_ml[at * 2 + 1] = l_run[r];
      }
      continue;
    }
    const float inv = l_run[r] > 0.f ? 1.f / l_run[r] : 0.f;
    __nv_bfloat16* dst = a.out + ((size_t)a.seq_qstart[seq] + row0) * a.n_heads * dv + (size_t)h * dv + row * o_stride;
#pragma unroll
    for (int n = 0; n < NT_OUT; ++n)
      if (n * 8 + 2 * t < dv)  // dv is even: a pair is inside or outside as a whole
        *reinterpret_cast<__nv_bfloat162*>(dst + n * 8 + 2 * t) =
            __floats2bfloat162_rn(o[n][2 * r] * inv, o[n][2 * r + 1] * inv);
  }
}

// out[seq, head, :] = sum_s o_s 2^(m_s - m) / sum_s l_s 2^(m_s - m) over the splits of a single-token step, in split order.
__global__ void local_mma_merge_kernel(LocalMmaArgs a) {
  const int seq = blockIdx.x / a.n_heads, head = blockIdx.x % a.n_heads;
  const size_t at = ((size_t)seq * a.n_heads + head) * a.n_splits;
  float m = -INFINITY;
  for (int s = 0; s < a.n_splits; ++s) m = fmaxf(m, a.part_ml[(at + s) * 2]);
  float l = 0.f;
  for (int s = 0; s < a.n_splits; ++s) {
    const float ms = a.part_ml[(at + s) * 2];
    if (ms > -INFINITY) l += a.part_ml[(at + s) * 2 + 1] * exp2f(ms - m);
  }
  const float inv = l > 0.f ? 1.f / l : 0.f;
  __nv_bfloat16* dst = a.out + (size_t)a.seq_qstart[seq] * a.n_heads * a.dv + (size_t)head * a.dv;
  for (int c = threadIdx.x; c < a.dv; c += blockDim.x) {
    float v = 0.f;
    for (int s = 0; s < a.n_splits; ++s) {
      const float ms = a.part_ml[(at + s) * 2];
      if (ms > -INFINITY) v += a.part_o[(at + s) * a.dv + c] * exp2f(ms - m);
    }
    dst[c] = __float2bfloat16_rn(v * inv);
  }
}

template <int DK, int DV>
int launch_local_mma(const LocalMmaArgs& a, int n_tiles, cudaStream_t stream) {
  const size_t smem = a.v_cache == a.k_cache ? (size_t)2 * LocalMmaSmem<DK, DV>::KTILE * 2 : LocalMmaSmem<DK, DV>::BYTES;
  auto kernel = local_prefill_mma_kernel<DK, DV>;
  cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (err != cudaSuccess) {
    mll_set_error("local attention (mma): cannot reserve %zu bytes of shared memory: %s", smem, cudaGetErrorString(err));
    return (int)err;
  }
  const int group = a.n_heads / a.n_kv_heads;
  const dim3 grid(n_tiles, a.heads_as_rows ? a.n_kv_heads * ((group + 63) / 64) : a.n_heads, a.n_splits);
  MLL_LAUNCH((kernel), grid, 128, smem, stream, a);
  MLL_LAUNCH_CHECK();
  if (a.n_splits > 1) {
    MLL_LAUNCH((local_mma_merge_kernel), n_tiles * a.n_heads, 64, 0, stream, a);
    MLL_LAUNCH_CHECK();
  }
  return 0;
}

template <int DK>
int dispatch_local_mma_v(const LocalMmaArgs& a, int n_tiles, cudaStream_t stream) {
  if (a.dv <= 32) return launch_local_mma<DK, 32>(a, n_tiles, stream);
  if (a.dv <= 64) return launch_local_mma<DK, 64>(a, n_tiles, stream);
  if (a.dv <= 128) return launch_local_mma<DK, 128>(a, n_tiles, stream);
  return launch_local_mma<DK, 256>(a, n_tiles, stream);
}

}  // namespace mll

MLL_API int mll_local_attention_mma_supported(int dtype, int d, int dv) {
  return dtype == MLL_BF16 && d >= 8 && d <= 256 && d % 8 == 0 && dv >= 8 && dv <= 256 && dv % 8 == 0;
}

// tile_seq / tile_row0: tiles of up to 64 query rows as (sequence, first row among the sequence's new tokens).
// heads_as_rows: every sequence brings one token; n_tiles is then the number of sequences and the lists are not read;
// n_splits > 1 cuts every context into that many runs of pages and needs scratch: n_tiles * n_heads * n_splits *
// (dv + 2) floats.
MLL_API int mll_local_attention_mma(const void* q, const void* k_cache, const void* v_cache, const int* seq_slot,
                                    const int* seq_ctx, const int* seq_qstart, const int* seq_qlen, const int* tile_seq,
                                    const int* tile_row0, const int* block_table, void* out, int n_tiles, int n_heads,
                                    int n_kv_heads, int d, int dv, int chunk, int window, int max_blocks, float scale,
                                    int sink, const float* sink_values, int v_in_k, int heads_as_rows, int n_splits,
                                    float* scratch, int keep_first, float softcap,
                                    cudaStream_t stream) {
  MLL_REQUIRE(mll_local_attention_mma_supported(MLL_BF16, d, dv), "local attention (mma): head sizes %d / %d", d, dv);
  MLL_REQUIRE(n_heads > 0 && n_kv_heads > 0 && n_heads % n_kv_heads == 0, "local attention (mma): bad head counts");
  MLL_REQUIRE(n_tiles >= 0 && n_heads <= 65535 && chunk >= 0 && window >= 0, "local attention (mma): bad tile count, chunk or window");
  MLL_REQUIRE(keep_first >= 0 && softcap >= 0.f && (keep_first == 0 || chunk == 0), "local attention (mma): bad kept tokens or cap");
  MLL_REQUIRE(!v_in_k || dv <= d, "local attention (mma): values of %d cannot be the leading columns of keys of %d", dv, d);
  MLL_REQUIRE(n_splits >= 1 && n_splits <= 64 && (n_splits == 1 || (heads_as_rows && scratch != nullptr)),
              "local attention (mma): %d context splits need single tokens and scratch memory", n_splits);
  if (n_tiles == 0) return 0;
  mll::LocalMmaArgs a{(const __nv_bfloat16*)q, (const __nv_bfloat16*)k_cache, (const __nv_bfloat16*)v_cache,
                      seq_slot, seq_ctx, seq_qstart, seq_qlen, tile_seq, tile_row0, block_table,
                      (__nv_bfloat16*)out, n_heads, n_kv_heads, max_blocks, window, chunk, d, dv,
                      scale * 1.4426950408889634f, (sink || sink_values) ? 1 : 0, sink_values, heads_as_rows ? 1 : 0, v_in_k ? d : dv, n_splits,
                      scratch, scratch ? scratch + (size_t)n_tiles * n_heads * n_splits * dv : nullptr, keep_first, softcap,
                      scale};
  if (d <= 32) return mll::dispatch_local_mma_v<32>(a, n_tiles, stream);
  if (d <= 64) return mll::dispatch_local_mma_v<64>(a, n_tiles, stream);
  if (d <= 128) return mll::dispatch_local_mma_v<128>(a, n_tiles, stream);
  return mll::dispatch_local_mma_v<256>(a, n_tiles, stream);
}
