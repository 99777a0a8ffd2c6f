// Attention whose keys and values have head sizes of their own (d for queries and keys, dv for
// values), with an explicit score scale, an optional norm of the whole q and k projections, rotary
// encoding of the first `rot` dimensions of a head only, and a mask that is causal inside chunks:
// query i sees key j iff j <= i and j / chunk == i / chunk (chunk 0: every earlier key), and with a
// window w > 0 only keys j > i - w.  Chunks count from position 0 of the sequence, whatever portion of it
// a step brings.  Two further options: a query temperature (q at position p is multiplied by
// 1 + coef * ln(floor((p + 1) / every) + 1) before it is stored) and a sink in the softmax (one more term
// exp(0) in the denominator that carries no value, so a row's weights may sum to less than one).  The values
// may be the leading dv columns of the key rows (v_ld = d: a layer that caches one latent row per position and
// reads it as key and as value); otherwise they have pages of their own (v_ld = dv).
// A window may keep the sequence's first tokens (`keep_first`: key j < keep_first stays visible whatever its distance, at
// its own position), and a score may be capped smoothly (s <- cap * tanh(s / cap) after the scale).  A layer that reads
// another layer's keys and values prepares its queries only (`write_kv` 0).
//
// Two kernels, for prompts and single tokens alike:
//   * prepare: one block per token.  q and k are each divided by the root mean square of their whole
//     projection (all heads at once) and multiplied by a weight, the pairs of the first `rot`
//     dimensions of every head are rotated by position * frequency (cos / sin from a table), q goes to
//     a buffer and k, v into the pages of the cache.  All arithmetic in float32.
//   * attend: one block per (token, kv head) and the query heads of its group.  Pages of keys and values pass
//     through shared memory; scores are float32 dot products over the head, the softmax runs online in
//     float32.  Any d and dv (16-byte copies where rows are whole 16-byte words).
#include "common.cuh"

namespace mll {

struct LocalPrepArgs {
  const void* qkv;        // [T, ld]: q (Hq * d), k (Hk * d), v (Hk * dv)
  const float* q_weight;  // [Hq * d] or null: no norm of the projections
  const float* k_weight;  // [Hk * d]
  const float* cos_table; // [max_pos, rot / 2] or null
  const float* sin_table;
  const int* tok_pos;
  const int* tok_seq;
  const int* seq_slot;
  const int* block_table;
  void* q_out;            // [T, Hq * d]
  void* k_cache;          // [pages, Hk, PAGE, d]
  void* v_cache;          // [pages, Hk, PAGE, dv]
  int ld, n_heads, n_kv_heads, d, dv, rot, interleaved, max_blocks;
  float eps;
  float q_temp_coef;      // query temperature: 0 and 0 for none
  int q_temp_every;
  int v_col;              // column of a row where the values begin: behind k, or k's own columns (values that are
                          // the keys as projected, before norm and rotation)
  int write_kv;           // 0: the row holds queries only; nothing goes to the cache (another layer's is read)
};

template <typename T>
__global__ void __launch_bounds__(256) local_prepare_kernel(LocalPrepArgs a) {
  __shared__ float scratch[32];
  const int t = blockIdx.x;
  const int d = a.d, nq = a.n_heads * d, nk = a.write_kv ? a.n_kv_heads * d : 0, nv = a.write_kv ? a.n_kv_heads * a.dv : 0;
  const T* row = (const T*)a.qkv + (size_t)t * a.ld;
  float fq = 1.f, fk = 1.f;
  if (a.q_weight) {
    float sq = 0.f, sk = 0.f;
    for (int i = threadIdx.x; i < nq; i += blockDim.x) {
      const float v = to_float(row[i]);
      sq += v * v;
    }
    for (int i = threadIdx.x; i < nk; i += blockDim.x) {
      const float v = to_float(row[nq + i]);
      sk += v * v;
    }
    sq = block_sum(sq, scratch);
    sk = block_sum(sk, scratch);
    fq = 1.f / sqrtf(sq / (float)nq + a.eps);
    fk = 1.f / sqrtf(sk / (float)nk + a.eps);
  }
  const int pos = a.tok_pos[t];
  if (a.q_temp_every > 0) fq *= 1.f + a.q_temp_coef * logf((float)((pos + 1) / a.q_temp_every) + 1.f);
  const int slot = a.seq_slot[a.tok_seq[t]];
  const int page = a.write_kv ? a.block_table[(size_t)slot * a.max_blocks + pos / MLL_PAGE] : 0;
  const int in_page = pos % MLL_PAGE;
  const int half = a.rot >> 1;
  const float* cs = a.cos_table ? a.cos_table + (size_t)pos * half : nullptr;
  const float* sn = a.cos_table ? a.sin_table + (size_t)pos * half : nullptr;
  for (int i = threadIdx.x; i < nq + nk; i += blockDim.x) {
    const bool is_q = i < nq;
    const int c = is_q ? i : i - nq;  // column within the q or k projection
    const int head = c / d, e = c % d;
    const float* w = is_q ? a.q_weight : a.k_weight;
    const float f = is_q ? fq : fk;
    const T* src = row + (is_q ? 0 : nq) + head * d;
    float x = to_float(src[e]) * f;
    if (w) x *= w[c];
    if (cs && e < a.rot) {
      int pair, partner;
      bool first;
      if (a.interleaved) {
        pair = e >> 1; first = !(e & 1); partner = e ^ 1;
      } else {
        first = e < half; pair = first ? e : e - half; partner = first ? e + half : e - half;
      }
      float y = to_float(src[partner]) * f;
      if (w) y *= w[head * d + partner];
      const float co = cs[pair], si = sn[pair];
      x = first ? x * co - y * si : x * co + y * si;
    }
    if (is_q)
      ((T*)a.q_out)[(size_t)t * nq + c] = from_float<T>(x);
    else
      ((T*)a.k_cache)[(((size_t)page * a.n_kv_heads + head) * MLL_PAGE + in_page) * d + e] = from_float<T>(x);
  }
  for (int i = threadIdx.x; i < nv; i += blockDim.x) {
    const int head = i / a.dv, e = i % a.dv;
    ((T*)a.v_cache)[(((size_t)page * a.n_kv_heads + head) * MLL_PAGE + in_page) * a.dv + e] = row[a.v_col + i];
  }
}

template <typename T>
struct Vec16;  // 16 bytes of T as floats
template <>
struct Vec16<float> {
  static __device__ __forceinline__ void load(const float* p, float* out) {
    const float4 v = *reinterpret_cast<const float4*>(p);
    out[0] = v.x; out[1] = v.y; out[2] = v.z; out[3] = v.w;
  }
};
template <>
struct Vec16<__nv_bfloat16> {
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float* out) {
    const uint4 v = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __bfloat1622float2(h[i]);
      out[2 * i] = f.x;
      out[2 * i + 1] = f.y;
    }
  }
};

struct LocalAttnArgs {
  const void* q;         // [T, Hq * d]
  const void* k_cache;
  const void* v_cache;
  const int* tok_pos;
  const int* tok_seq;
  const int* seq_slot;
  const int* block_table;
  void* out;             // [T, Hq * dv]
  int n_tokens, n_heads, n_kv_heads, d, dv, chunk, window, max_blocks;
  float scale;
  int sink;              // 1: the softmax's denominator has one more term exp(sink value)
  const float* sink_values;  // [Hq] the sink's score per query head (unscaled), or null: 0
  int v_ld;              // elements between value rows: dv, or d when the values are the keys' leading columns
  int keep_first;        // with a window: keys at positions below this stay visible
  float softcap;         // > 0: score <- softcap * tanh(score / softcap)
};

// grid (tokens, Hk * head chunks), 128 threads.  A block owns one token, one kv head and up to `hpb` of the
// query heads that read it; it walks the pages that hold keys first .. pos.  A page's keys and values are
// brought into shared memory by all threads (16-byte asynchronous copies where rows are whole 16-byte words,
// two pages in flight where shared memory allows), so that the loads of a page are all in flight together
// and every key and value is read once for the heads of its group.
template <typename T, int NACC>
__global__ void __launch_bounds__(128) local_attention_kernel(LocalAttnArgs a, int hpb, int stages, int vec) {
  const int d = a.d, dv = a.dv;
  const int group = a.n_heads / a.n_kv_heads;
  const int chunks = (group + hpb - 1) / hpb;
  const int t = blockIdx.x;
  const int kvh = blockIdx.y / chunks, g0 = (blockIdx.y % chunks) * hpb;
  const int ng = min(hpb, group - g0);
  const int h0 = kvh * group + g0;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int pos = a.tok_pos[t];
  int first = a.chunk > 0 ? (pos / a.chunk) * a.chunk : 0;
  if (a.window > 0) first = max(first, pos - a.window + 1);
  const int* table = a.block_table + (size_t)a.seq_slot[a.tok_seq[t]] * a.max_blocks;

  extern __shared__ __align__(16) unsigned char smem_raw[];
  constexpr int PAD = 16 / sizeof(T);
  const int d_pad = (d + 3) & ~3;
  float* q_s = reinterpret_cast<float*>(smem_raw);   // [hpb][d_pad], scaled
  float* s_s = q_s + hpb * d_pad;                     // [hpb][PAGE]
  float* m_s = s_s + hpb * MLL_PAGE;                  // [hpb] running maximum, sum, rescale factor
  float* l_s = m_s + hpb;
  float* alpha_s = l_s + hpb;
  size_t off = (size_t)((alpha_s + hpb) - q_s) * sizeof(float);
  off = (off + 15) & ~(size_t)15;
  const int k_stride = ((d + PAD - 1) / PAD) * PAD + PAD;  // elements; rows start on 16-byte boundaries
  const int v_stride = ((dv + PAD - 1) / PAD) * PAD;
  const size_t k_tile = (size_t)MLL_PAGE * k_stride, v_tile = (size_t)MLL_PAGE * v_stride;
  T* k_s = reinterpret_cast<T*>(smem_raw + off);
  T* v_s = k_s + stages * k_tile;

  for (int i = tid; i < ng * d; i += 128) {
    const int g = i / d, e = i % d;
    q_s[g * d_pad + e] = to_float(((const T*)a.q)[((size_t)t * a.n_heads + h0 + g) * d + e]) * a.scale;
  }
  for (int i = tid; i < ng; i += 128) {
    // the sink: a key with a score of its own and no value, seen before all others
    m_s[i] = a.sink ? (a.sink_values ? a.sink_values[h0 + i] : 0.f) : -INFINITY;
    l_s[i] = a.sink ? 1.f : 0.f;
  }
  float acc[NACC];
#pragma unroll
  for (int i = 0; i < NACC; ++i) acc[i] = 0.f;

  const int p_begin = first / MLL_PAGE, p_end = pos / MLL_PAGE + 1;
  // the kept first tokens that lie in front of the window: keys [0, kept), on the pages in front of p_begin and on
  // p_begin itself (whose rows between `kept` and `first` are then skipped)
  const int kept = (a.window > 0 && a.keep_first > 0) ? min(a.keep_first, first) : 0;
  const int n_kept_pages = min((kept + MLL_PAGE - 1) / MLL_PAGE, p_begin);  // walked before p_begin
  auto page_of = [&](int walk) { return walk < n_kept_pages ? walk : p_begin + (walk - n_kept_pages); };
  const int n_walk = n_kept_pages + (p_end - p_begin);
  auto load_tiles = [&](int page_index, int stage) {
    const int page = table[page_index];
    const T* kg = (const T*)a.k_cache + ((size_t)page * a.n_kv_heads + kvh) * MLL_PAGE * d;
    const T* vg = (const T*)a.v_cache + ((size_t)page * a.n_kv_heads + kvh) * MLL_PAGE * a.v_ld;
    T* kd = k_s + stage * k_tile;
    T* vd = v_s + stage * v_tile;
    // every row up to the last visible one is loaded when kept keys share the page; the scores mask the gap
    const int r_lo = page_index * MLL_PAGE < kept ? 0 : max(0, first - page_index * MLL_PAGE);
    const int r_hi = min(MLL_PAGE, pos + 1 - page_index * MLL_PAGE);
    if (vec) {
      const int kc = d / PAD, vc = dv / PAD;
      for (int c = tid; c < (r_hi - r_lo) * kc; c += 128) {
        const int r = r_lo + c / kc, cc = c % kc;
        cp_async16(kd + (size_t)r * k_stride + cc * PAD, kg + (size_t)r * d + cc * PAD);
      }
      for (int c = tid; c < (r_hi - r_lo) * vc; c += 128) {
        const int r = r_lo + c / vc, cc = c % vc;
        cp_async16(vd + (size_t)r * v_stride + cc * PAD, vg + (size_t)r * a.v_ld + cc * PAD);
      }
    } else {
      for (int c = tid; c < (r_hi - r_lo) * d; c += 128) {
        const int r = r_lo + c / d, e = c % d;
        kd[(size_t)r * k_stride + e] = kg[(size_t)r * d + e];
      }
      for (int c = tid; c < (r_hi - r_lo) * dv; c += 128) {
        const int r = r_lo + c / dv, e = c % dv;
        vd[(size_t)r * v_stride + e] = vg[(size_t)r * a.v_ld + e];
      }
    }
  };

  load_tiles(page_of(0), 0);
  cp_async_commit();
  for (int it = 0; it < n_walk; ++it) {
    const int p = page_of(it);
    const int cur = stages == 2 ? (it & 1) : 0;
    if (stages == 2 && it + 1 < n_walk) {
      load_tiles(page_of(it + 1), cur ^ 1);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const T* kt = k_s + cur * k_tile;
    const T* vt = v_s + cur * v_tile;
    const int jlo = p * MLL_PAGE < kept ? 0 : max(0, first - p * MLL_PAGE), jhi = min(MLL_PAGE, pos + 1 - p * MLL_PAGE);

    for (int idx = tid; idx < ng * MLL_PAGE; idx += 128) {
      const int g = idx / MLL_PAGE, j = idx % MLL_PAGE;
      float sc = -INFINITY;
      const int kpos = p * MLL_PAGE + j;
      if (j >= jlo && j < jhi && (kpos >= first || kpos < kept)) {
        const T* kr = kt + (size_t)j * k_stride;
        const float* qg = q_s + g * d_pad;
        float dot = 0.f;
        if (vec) {
          for (int e = 0; e < d; e += PAD) {
            float kv[PAD];
            Vec16<T>::load(kr + e, kv);
#pragma unroll
            for (int u = 0; u < PAD; ++u) dot = fmaf(qg[e + u], kv[u], dot);
          }
        } else {
          for (int e = 0; e < d; ++e) dot = fmaf(qg[e], to_float(kr[e]), dot);
        }
        sc = a.softcap > 0.f ? a.softcap * tanhf(dot / a.softcap) : dot;
      }
      s_s[idx] = sc;
    }
    __syncthreads();
    for (int g = warp; g < ng; g += 4) {
      const float v0 = s_s[g * MLL_PAGE + lane], v1 = s_s[g * MLL_PAGE + lane + 32];
      const float m_old = m_s[g];
      const float m_new = fmaxf(m_old, warp_max(fmaxf(v0, v1)));  // every page of the walk holds a visible key: finite
      const float alpha = expf(m_old - m_new);
      const float p0 = expf(v0 - m_new), p1 = expf(v1 - m_new);
      s_s[g * MLL_PAGE + lane] = p0;
      s_s[g * MLL_PAGE + lane + 32] = p1;
      const float psum = warp_sum(p0 + p1);
      if (lane == 0) {
        l_s[g] = l_s[g] * alpha + psum;
        m_s[g] = m_new;
        alpha_s[g] = alpha;
      }
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < NACC; ++i) {
      const int o = tid + 128 * i;
      if (o < ng * dv) {
        const int g = o / dv, e = o % dv;
        float v = acc[i] * alpha_s[g];
        const float* pg = s_s + g * MLL_PAGE;
        for (int j = jlo; j < jhi; ++j) v = fmaf(pg[j], to_float(vt[(size_t)j * v_stride + e]), v);
        acc[i] = v;
      }
    }
    __syncthreads();
    if (stages == 1 && it + 1 < n_walk) {
      load_tiles(page_of(it + 1), 0);
      cp_async_commit();
    }
  }
#pragma unroll
  for (int i = 0; i < NACC; ++i) {
    const int o = tid + 128 * i;
    if (o < ng * dv) {
      const float l = l_s[o / dv];
      ((T*)a.out)[((size_t)t * a.n_heads + h0) * dv + o] = from_float<T>(l > 0.f ? acc[i] / l : 0.f);
    }
  }
}

template <typename T>
int launch_local_attention(const LocalAttnArgs& a, cudaStream_t stream) {
  constexpr int PAD = 16 / sizeof(T);
  const int group = a.n_heads / a.n_kv_heads;
  const int hpb = max(1, min(group, 1024 / a.dv));       // at most 8 accumulators a thread
  const int chunks = (group + hpb - 1) / hpb;
  const int vec = (a.d % PAD == 0 && a.dv % PAD == 0 && a.v_ld % PAD == 0) ? 1 : 0;
  const int k_stride = ((a.d + PAD - 1) / PAD) * PAD + PAD, v_stride = ((a.dv + PAD - 1) / PAD) * PAD;
  size_t fixed = (size_t)(hpb * ((a.d + 3) & ~3) + hpb * MLL_PAGE + 3 * hpb) * sizeof(float);
  fixed = (fixed + 15) & ~(size_t)15;
  const size_t tile = (size_t)MLL_PAGE * (k_stride + v_stride) * sizeof(T);
  const int stages = fixed + 2 * tile <= 96 * 1024 ? 2 : 1;
  const size_t smem = fixed + stages * tile;
  MLL_REQUIRE(smem <= 200 * 1024, "local attention: head sizes %d / %d need %zu bytes of shared memory", a.d, a.dv, smem);
  MLL_REQUIRE((long long)a.n_kv_heads * chunks <= 65535, "local attention: too many heads for one launch");
  const dim3 grid(a.n_tokens, a.n_kv_heads * chunks);
  const int nacc = (hpb * a.dv + 127) / 128;
#define MLL_LOCAL_LAUNCH(N)                                                                                   \
  do {                                                                                                        \
    auto kernel = local_attention_kernel<T, N>;                                                               \
    if (smem > 48 * 1024) {                                                                                   \
      cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
      if (err != cudaSuccess) {                                                                               \
        mll_set_error("local attention: cannot reserve %zu bytes of shared memory: %s", smem,                 \
                      cudaGetErrorString(err));                                                               \
        return (int)err;                                                                                      \
      }                                                                                                       \
    }                                                                                                         \
    MLL_LAUNCH((kernel), grid, 128, smem, stream, a, hpb, stages, vec);                                       \
  } while (0)
  if (nacc <= 1) MLL_LOCAL_LAUNCH(1);
  else if (nacc <= 2) MLL_LOCAL_LAUNCH(2);
  else if (nacc <= 4) MLL_LOCAL_LAUNCH(4);
  else MLL_LOCAL_LAUNCH(8);
#undef MLL_LOCAL_LAUNCH
  MLL_LAUNCH_CHECK();
  return 0;
}

}  // namespace mll

MLL_API int mll_local_attention_prepare(const void* qkv, const float* q_weight, const float* k_weight,
                                        const float* cos_table, const float* sin_table, const int* tok_pos,
                                        const int* tok_seq, const int* seq_slot, const int* block_table, void* q_out,
                                        void* k_cache, void* v_cache, int dtype, int n_tokens, int ld, int n_heads,
                                        int n_kv_heads, int d, int dv, int rot, int interleaved, int max_blocks,
                                        float eps, float q_temp_coef, int q_temp_every, int v_from_k, int write_kv,
                                        cudaStream_t stream) {
  MLL_REQUIRE(n_tokens >= 0 && n_heads > 0 && n_kv_heads > 0 && d > 0 && dv > 0, "local attention prepare: bad sizes");
  MLL_REQUIRE(rot >= 0 && rot <= d && rot % 2 == 0, "local attention prepare: %d rotated dimensions of %d", rot, d);
  MLL_REQUIRE((q_weight == nullptr) == (k_weight == nullptr), "local attention prepare: one norm weight without the other");
  MLL_REQUIRE(ld >= n_heads * d + (write_kv ? n_kv_heads * (v_from_k ? d : d + dv) : 0), "local attention prepare: row stride %d too short", ld);
  MLL_REQUIRE(!v_from_k || dv == d, "local attention prepare: values that are the keys need dv == d, got %d / %d", dv, d);
  MLL_REQUIRE(q_temp_every >= 0, "local attention prepare: negative temperature period");
  if (n_tokens == 0) return 0;
  mll::LocalPrepArgs a{qkv, q_weight, k_weight, rot > 0 ? cos_table : nullptr, sin_table, tok_pos, tok_seq, seq_slot,
                       block_table, q_out, k_cache, v_cache, ld, n_heads, n_kv_heads, d, dv, rot, interleaved,
                       max_blocks, eps, q_temp_coef, q_temp_every,
                       v_from_k ? n_heads * d : n_heads * d + n_kv_heads * d, write_kv ? 1 : 0};
  if (dtype == MLL_F32)
    MLL_LAUNCH((mll::local_prepare_kernel<float>), n_tokens, 256, 0, stream, a);
  else if (dtype == MLL_BF16)
    MLL_LAUNCH((mll::local_prepare_kernel<__nv_bfloat16>), n_tokens, 256, 0, stream, a);
  else
    MLL_REQUIRE(false, "local attention prepare: unknown dtype %d", dtype);
  MLL_LAUNCH_CHECK();
  return 0;
}

MLL_API int mll_local_attention(const void* q, const void* k_cache, const void* v_cache, const int* tok_pos,
                                const int* tok_seq, const int* seq_slot, const int* block_table, void* out, int dtype,
                                int n_tokens, int n_heads, int n_kv_heads, int d, int dv, int chunk, int window,
                                int max_blocks, float scale, int sink, const float* sink_values, int v_in_k,
                                int keep_first, float softcap, cudaStream_t stream) {
  MLL_REQUIRE(n_tokens >= 0 && n_heads > 0 && n_kv_heads > 0 && n_heads % n_kv_heads == 0, "local attention: bad head counts");
  MLL_REQUIRE(d > 0 && d <= 1024 && dv > 0 && dv <= 1024, "local attention: head sizes %d / %d (at most 1024)", d, dv);
  MLL_REQUIRE(chunk >= 0 && window >= 0 && keep_first >= 0 && softcap >= 0.f, "local attention: negative chunk, window, kept tokens or cap");
  MLL_REQUIRE(keep_first == 0 || chunk == 0, "local attention: kept first tokens go with a window, not with chunks");
  MLL_REQUIRE(!v_in_k || dv <= d, "local attention: values of %d cannot be the leading columns of keys of %d", dv, d);
  if (n_tokens == 0) return 0;
  mll::LocalAttnArgs a{q, k_cache, v_cache, tok_pos, tok_seq, seq_slot, block_table, out, n_tokens, n_heads,
                       n_kv_heads, d, dv, chunk, window, max_blocks, scale, (sink || sink_values) ? 1 : 0, sink_values,
                       v_in_k ? d : dv, keep_first, softcap};
  if (dtype == MLL_F32) return mll::launch_local_attention<float>(a, stream);
  if (dtype == MLL_BF16) return mll::launch_local_attention<__nv_bfloat16>(a, stream);
  MLL_REQUIRE(false, "local attention: unknown dtype %d", dtype);
  return -1;
}
