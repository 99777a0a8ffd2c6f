// Mixers that carry a matrix-valued state per sequence and head instead of keys and values:
//
//   S_t = diag(g_t) S_(t-1) + k_t u_t^T,      o_t = S_t^T q_t          S is [d, dv], float32
//
// with  u_t = v_t                              and one fixed decay per head      ("retention"), or
//       u_t = beta_t (v_t - (diag(g_t) S_(t-1))^T k_t), g_t per key channel      (the gated delta rule), or
//       u_t = v_t                              and g_t per key channel           (gated linear attention).
// The read-out sees the current token's write.  Everything that enters the recurrence is float32.
//
// Kernels (each for prompts and single tokens alike; a step's tokens of one sequence are consecutive rows):
//   * retention_prepare   rotary encoding of q and k (first `rot` dimensions of a head), k / sqrt(d); q, k, v
//                         to float32
//   * delta_prepare       short causal convolution over time + silu on q, k, v (the inputs before this step's
//                         first token come from the sequence's state), q and k to unit length per head,
//                         q / sqrt(d), beta = sigmoid, g = exp(-exp(A) softplus(x + bias))
//   * channel_decay_prepare  q * q_scale, k, v to float32 and g = sigmoid(z + bias)^(1 / tau) per key channel,
//                         formed as exp(log_sigmoid(z + bias) / tau) in float32
//   * ssd_prepare         a state-space layer's inputs: short causal convolution with bias + silu on (x, B, C),
//                         dt = softplus(dt + bias), decay = exp(-exp(A) dt) per token and head, u = dt x
//   * conv_state_update   the last taps - 1 convolution inputs of every sequence, kept for the next step
//   * state_scan          the recurrence: a column of S lives in the registers of R lanes (ROWS rows each);
//                         per token every product is local to the column, two shuffles-reductions over the
//                         R lanes give S^T k and S^T q
//   * head_norm_gate      o / rms(o) per head (* weight) * silu or sigmoid of a gate, to the activation dtype
//   * gated_group_norm    (o + skip_h x) * silu(z), then / rms over each of a few equal parts of the row, * weight
#include "common.cuh"

namespace mll {

__device__ __forceinline__ float silu_f(float z) { return z / (1.f + expf(-z)); }
__device__ __forceinline__ float sigmoid_f(float z) { return 1.f / (1.f + expf(-z)); }
__device__ __forceinline__ float softplus_f(float z) { return z > 20.f ? z : log1pf(expf(z)); }

// ---------------------------------------------------------------------------------------------- //
struct RetPrepArgs {
  const void* proj;   // [T, ld]: q (H * d), k (H * d), v (H * dv), then whatever else
  const float* cos_table;
  const float* sin_table;
  const int* tok_pos;
  float* q;           // [T, H, d]
  float* k;
  float* v;           // [T, H, dv]
  int ld, n_heads, d, dv, rot, interleaved;
  float k_scale;
};

template <typename T>
__global__ void __launch_bounds__(256) retention_prepare_kernel(RetPrepArgs a) {
  const int t = blockIdx.x;
  const int d = a.d, n = a.n_heads * d, nv = a.n_heads * a.dv;
  const T* row = (const T*)a.proj + (size_t)t * a.ld;
  const int pos = a.tok_pos[t];
  const int half = a.rot >> 1;
  const float* cs = a.cos_table ? a.cos_table + (size_t)pos * half : nullptr;
  const float* sn = a.cos_table ? a.sin_table + (size_t)pos * half : nullptr;
  for (int i = threadIdx.x; i < 2 * n; i += blockDim.x) {
    const bool is_q = i < n;
    const int c = is_q ? i : i - n;
    const int head = c / d, e = c % d;
    const T* src = row + (is_q ? 0 : n) + head * d;
    float x = to_float(src[e]);
    if (cs && e < a.rot) {
      int pair, partner;
      bool first;
      if (a.interleaved) {
        pair = e >> 1; first = !(e & 1); partner = e ^ 1;
      } else {
        first = e < half; pair = first ? e : e - half; partner = first ? e + half : e - half;
      }
      const float y = to_float(src[partner]);
      const float co = cs[pair], si = sn[pair];
      x = first ? x * co - y * si : x * co + y * si;
    }
    if (is_q)
      a.q[(size_t)t * n + c] = x;
    else
      a.k[(size_t)t * n + c] = x * a.k_scale;
  }
  for (int i = threadIdx.x; i < nv; i += blockDim.x) a.v[(size_t)t * nv + i] = to_float(row[2 * n + i]);
}

// ---------------------------------------------------------------------------------------------- //
struct DeltaPrepArgs {
  const void* proj;        // [T, ld]: q (G * d), k (G * d), v (H * dv), beta (H)
  const float* rate;       // [T, rate_ld]: the decay's pre-activation (H * d), float32
  const float* conv_w;     // [C, taps], C = 2 G d + H dv, rows in the order of proj's columns
  const float* conv_state; // [slots, taps - 1, C]
  const float* a_log;      // [H]
  const float* dt_bias;    // [H * d]
  const int* tok_seq;
  const int* seq_slot;
  const int* seq_qstart;
  float* q;                // [T, G, d]
  float* k;
  float* v;                // [T, H, dv]
  float* g;                // [T, H, d]
  float* beta;             // [T, H]
  int ld, rate_ld, n_heads, n_kv_heads, d, dv, taps;
  float unit_eps;
};

// grid (ceil(tokens / 4), 2 G + H), 128 threads: a warp owns one head of one token - a q head, a k head, or a
// value head together with that head's beta and decays - so that nothing waits on a block-wide barrier and a
// multiprocessor has many independent chains of loads in flight.  Dynamic shared memory: 4 * max(d, dv) floats.
template <typename T>
__global__ void __launch_bounds__(128) delta_prepare_kernel(DeltaPrepArgs a, int n_tokens) {
  extern __shared__ float conv_all[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * 4 + warp, unit = blockIdx.y;
  if (t >= n_tokens) return;  // whole warps leave; nothing below synchronises the block
  const int H = a.n_heads, G = a.n_kv_heads, d = a.d, dv = a.dv, taps = a.taps;
  float* conv_out = conv_all + warp * max(d, dv);
  const int nqk = G * d, C = 2 * nqk + H * dv;
  const int seq = a.tok_seq[t];
  const int local = t - a.seq_qstart[seq];  // index among this step's tokens of the sequence
  const float* state = a.conv_state + (size_t)a.seq_slot[seq] * (taps - 1) * C;
  const T* proj = (const T*)a.proj;
  const bool is_v = unit >= 2 * G;
  const int width = is_v ? dv : d;
  const int c0 = is_v ? 2 * nqk + (unit - 2 * G) * dv : unit * d;  // first channel of the head
  float ss = 0.f;
  for (int e = lane; e < width; e += 32) {
    const int c = c0 + e;
    float y = 0.f;
    for (int back = 0; back < taps; ++back) {  // the input `back` tokens ago meets tap taps - 1 - back
      float x;
      if (back <= local)
        x = to_float(proj[(size_t)(t - back) * a.ld + c]);
      else
        x = state[(size_t)(local - back + taps - 1) * C + c];
      y = fmaf(a.conv_w[(size_t)c * taps + (taps - 1 - back)], x, y);
    }
    y = silu_f(y);
    conv_out[e] = y;
    ss += y * y;
  }
  if (is_v) {
    const int h = unit - 2 * G;
    for (int e = lane; e < dv; e += 32) a.v[((size_t)t * H + h) * dv + e] = conv_out[e];
    if (lane == 0) a.beta[(size_t)t * H + h] = sigmoid_f(to_float(proj[(size_t)t * a.ld + C + h]));
    const float rate = expf(a.a_log[h]);
    for (int e = lane; e < d; e += 32) {
      const float sp = softplus_f(a.rate[(size_t)t * a.rate_ld + h * d + e] + a.dt_bias[h * d + e]);
      a.g[((size_t)t * H + h) * d + e] = expf(-rate * sp);
    }
    return;
  }
  ss = warp_sum(ss);  // q and k heads: unit length (and q / sqrt(d))
  const bool is_q = unit < G;
  const float f = (is_q ? rsqrtf((float)d) : 1.f) / sqrtf(ss + a.unit_eps);
  float* dst = (is_q ? a.q : a.k) + ((size_t)t * G + (is_q ? unit : unit - G)) * d;
  for (int e = lane; e < d; e += 32) dst[e] = conv_out[e] * f;
}

// grid (tokens), 256 threads: q * q_scale, k, v of a layer whose decay is sigmoid(z + bias)^(1 / tau) per key channel.
struct ChannelDecayArgs {
  const void* proj;    // [T, ld]: q (H * d), k (H * d), v (H * dv), then whatever else
  const float* rate;   // [T, rate_ld]: z (H * d), float32
  const float* bias;   // [H * d] or null
  float* q;            // [T, H, d]
  float* k;
  float* v;            // [T, H, dv]
  float* g;            // [T, H, d]
  int ld, rate_ld, n_heads, d, dv;
  float q_scale, inv_tau;
};

template <typename T>
__global__ void __launch_bounds__(256) channel_decay_prepare_kernel(ChannelDecayArgs a) {
  const int t = blockIdx.x;
  const int n = a.n_heads * a.d, nv = a.n_heads * a.dv;
  const T* row = (const T*)a.proj + (size_t)t * a.ld;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    a.q[(size_t)t * n + i] = to_float(row[i]) * a.q_scale;
    a.k[(size_t)t * n + i] = to_float(row[n + i]);
    const float z = a.rate[(size_t)t * a.rate_ld + i] + (a.bias ? a.bias[i] : 0.f);
    // log(sigmoid(z)) = -softplus(-z), without cancellation on either side
    a.g[(size_t)t * n + i] = expf(-softplus_f(-z) * a.inv_tau);
  }
  for (int i = threadIdx.x; i < nv; i += blockDim.x) a.v[(size_t)t * nv + i] = to_float(row[2 * n + i]);
}

// A state-space layer's inputs.  A row of proj is [z (H dv) | x (H dv) | B (G d) | C (G d) | dt (H)]; x, B and C
// pass a causal convolution over time (taps per channel, the last one meets the current token; the inputs before a
// step's first token come from the sequence's state) with a bias and silu.
//   dt_h = softplus(dt_h + dt_bias_h)   decay[t, h] = exp(-exp(A_h) dt_h)   u[t, h, :] = dt_h x[t, h, :]
//   k = B, q = C (per group), xs = x after the convolution (for the skip).  All float32.
struct SsdPrepArgs {
  const void* proj;        // [T, ld]
  const float* conv_w;     // [C, taps], C = H dv + 2 G d
  const float* conv_b;     // [C]
  const float* conv_state; // [slots, taps - 1, C]
  const float* a_log;      // [H]
  const float* dt_bias;    // [H]
  const int* tok_seq;
  const int* seq_slot;
  const int* seq_qstart;
  float* q;                // [T, G, d]
  float* k;                // [T, G, d]
  float* u;                // [T, H, dv]
  float* xs;               // [T, H, dv]
  float* decay;            // [T, H]
  int ld, n_heads, n_groups, d, dv, taps;
};

// grid (tokens, pieces of the channels), 256 threads, a channel a thread; dynamic shared memory: H floats (dt per head).
// A block forms the step sizes of the heads whose x-channels it holds; the blocks of piece 0 also write the decays.
template <typename T>
__global__ void __launch_bounds__(256) ssd_prepare_kernel(SsdPrepArgs a, int per_block) {
  extern __shared__ float dt_s[];
  const int t = blockIdx.x;
  const int H = a.n_heads, G = a.n_groups, d = a.d, dv = a.dv, taps = a.taps;
  const int inner = H * dv, gn = G * d, C = inner + 2 * gn;
  const T* proj = (const T*)a.proj;
  const T* row = proj + (size_t)t * a.ld;
  const int c_begin = blockIdx.y * per_block, c_end = min(C, c_begin + per_block);
  const int h_begin = blockIdx.y == 0 ? 0 : min(H, c_begin / dv);
  const int h_end = blockIdx.y == 0 ? H : min(H, (min(c_end, inner) + dv - 1) / dv);
  for (int h = h_begin + threadIdx.x; h < h_end; h += blockDim.x) {
    const float dt = softplus_f(to_float(row[inner + C + h]) + a.dt_bias[h]);
    dt_s[h] = dt;
    if (blockIdx.y == 0) a.decay[(size_t)t * H + h] = expf(-expf(a.a_log[h]) * dt);
  }
  __syncthreads();
  const int seq = a.tok_seq[t];
  const int local = t - a.seq_qstart[seq];  // index among this step's tokens of the sequence
  const float* state = a.conv_state + (size_t)a.seq_slot[seq] * (taps - 1) * C;
  for (int c = c_begin + threadIdx.x; c < c_end; c += blockDim.x) {
    float y = a.conv_b[c];
    for (int back = 0; back < taps; ++back) {  // the input `back` tokens ago meets tap taps - 1 - back
      float x;
      if (back <= local)
        x = to_float(proj[(size_t)(t - back) * a.ld + inner + c]);
      else
        x = state[(size_t)(local - back + taps - 1) * C + c];
      y = fmaf(a.conv_w[(size_t)c * taps + (taps - 1 - back)], x, y);
    }
    y = silu_f(y);
    if (c < inner) {
      a.xs[(size_t)t * inner + c] = y;
      a.u[(size_t)t * inner + c] = dt_s[c / dv] * y;
    } else if (c < inner + gn) {
      a.k[(size_t)t * gn + (c - inner)] = y;
    } else {
      a.q[(size_t)t * gn + (c - inner - gn)] = y;
    }
  }
}

// grid (ceil(C / 128), sequences): new state = the last taps - 1 of (old state, this step's inputs)
template <typename T>
__global__ void conv_state_update_kernel(const T* __restrict__ proj_rows, int col0, int ld, float* __restrict__ conv_state,
                                         const int* __restrict__ seq_slot, const int* __restrict__ seq_qstart,
                                         const int* __restrict__ seq_qlen, int C, int taps) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const T* proj = proj_rows + col0;  // the convolution's channels begin at column col0 of a row
  const int seq = blockIdx.y;
  const int n = seq_qlen[seq], row0 = seq_qstart[seq], keep = taps - 1;
  float* state = conv_state + (size_t)seq_slot[seq] * keep * C;
  if (n >= keep) {
    for (int i = 0; i < keep; ++i) state[(size_t)i * C + c] = to_float(proj[(size_t)(row0 + n - keep + i) * ld + c]);
  } else {
    for (int i = 0; i < keep - n; ++i) state[(size_t)i * C + c] = state[(size_t)(i + n) * C + c];  // ascending: reads run ahead of writes
    for (int i = 0; i < n; ++i) state[(size_t)(keep - n + i) * C + c] = to_float(proj[(size_t)(row0 + i) * ld + c]);
  }
}

// ---------------------------------------------------------------------------------------------- //
struct ScanArgs {
  const float* q;           // [T, G, d]
  const float* k;           // [T, G, d]
  const float* v;           // [T, H, dv]
  const float* g;           // [T, H, d] (a decay per key channel) or null
  const float* beta;        // [T, H]: the delta rule's beta, or (MODE 3) one decay per token and head; else null
  const float* head_decay;  // [H] (not DELTA)
  float* state;             // [slots, H, d, dv]
  float* out;               // [T, H, dv]
  const int* seq_slot;
  const int* seq_qstart;
  const int* seq_qlen;
  int n_heads, n_kv_heads, d, dv, tok_stage;
};

constexpr int SCAN_THREADS = 64;

__device__ __forceinline__ void cp_async4(float* smem, const float* gmem) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"(s), "l"(gmem));
}

// grid (column tiles, H, sequences).  Lane layout inside a warp: lane = r * (32 / R) + c; lane (r, c) holds rows
// r * ROWS .. r * ROWS + ROWS - 1 of column c of the warp's columns.  Rows past d are padding: their k and q
// are staged as 0, so their S stays 0 and adds nothing.  The tokens' q, k, g, v and beta arrive in shared memory
// `tok_stage` tokens at a time through a two-stage ring of asynchronous copies, so that the next tokens load
// while these are worked on and the chain from token to token is arithmetic only.
// MODE 0: one decay per head; 1: the delta rule with a decay per key channel; 2: a decay per key channel, u = v;
// 3: one decay per token and head (it travels where the delta rule's beta does), u = v.
template <int ROWS, int R, int MODE, int THREADS>
__global__ void __launch_bounds__(THREADS) state_scan_kernel(ScanArgs a) {
  constexpr bool DELTA = MODE == 1;    // beta and the correction by S^T k
  constexpr bool CHANNEL = MODE == 1 || MODE == 2;  // g per key channel travels with q and k
  constexpr bool TOKEN_DECAY = MODE == 3;
  extern __shared__ __align__(16) float stage[];
  constexpr int DP = ROWS * R;          // padded number of rows
  constexpr int CPW = 32 / R;           // columns per warp
  constexpr int CPB = CPW * (THREADS / 32);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int r = lane / CPW, cw = lane % CPW;
  const int col0 = blockIdx.x * CPB;
  const int col = col0 + warp * CPW + cw;
  const int h = blockIdx.y, seq = blockIdx.z;
  const int H = a.n_heads, G = a.n_kv_heads, d = a.d, dv = a.dv;
  const int kvh = h / (H / G);
  const int row0 = a.seq_qstart[seq], n_tok = a.seq_qlen[seq];
  const bool live = col < dv;
  float* S = a.state + (((size_t)a.seq_slot[seq] * H + h) * d) * dv;
  float s[ROWS];
#pragma unroll
  for (int i = 0; i < ROWS; ++i) {
    const int row = r * ROWS + i;
    s[i] = (live && row < d) ? S[(size_t)row * dv + col] : 0.f;
  }
  const int TS = a.tok_stage;
  const int per_stage = (TS * DP * (CHANNEL ? 3 : 2) + TS * CPB + TS + 3) & ~3;  // stages start on 16-byte boundaries
  // the padding rows of both stages, once: the copies below never touch them
  if (d < DP)
  for (int i = tid; i < 2 * TS * DP; i += THREADS) {
    const int st = i / (TS * DP), rest = i % (TS * DP);
    if (rest % DP >= d) {
      float* base = stage + st * per_stage;
      base[rest] = 0.f;
      base[TS * DP + rest] = 0.f;
      if (CHANNEL) base[2 * TS * DP + rest] = 1.f;
    }
  }
  auto load = [&](int t0, int st) {
    const int nt = min(TS, n_tok - t0);
    float* q_s = stage + st * per_stage;
    float* k_s = q_s + TS * DP;
    float* g_s = k_s + TS * DP;
    float* v_s = stage + st * per_stage + TS * DP * (CHANNEL ? 3 : 2);
    float* b_s = v_s + TS * CPB;
    if ((d & 3) == 0) {  // rows are whole 16-byte words
      const int words = d >> 2;
      for (int i = tid; i < nt * words; i += THREADS) {
        const int tt = i / words, e = (i % words) << 2;
        const size_t tok = (size_t)(row0 + t0 + tt);
        cp_async16(q_s + tt * DP + e, a.q + (tok * G + kvh) * d + e);
        cp_async16(k_s + tt * DP + e, a.k + (tok * G + kvh) * d + e);
        if (CHANNEL) cp_async16(g_s + tt * DP + e, a.g + (tok * H + h) * d + e);
      }
    } else {
      for (int i = tid; i < nt * d; i += THREADS) {
        const int tt = i / d, e = i % d;
        const size_t tok = (size_t)(row0 + t0 + tt);
        cp_async4(q_s + tt * DP + e, a.q + (tok * G + kvh) * d + e);
        cp_async4(k_s + tt * DP + e, a.k + (tok * G + kvh) * d + e);
        if (CHANNEL) cp_async4(g_s + tt * DP + e, a.g + (tok * H + h) * d + e);
      }
    }
    for (int i = tid; i < nt * CPB; i += THREADS) {
      const int tt = i / CPB, c = i % CPB;
      if (col0 + c < dv) cp_async4(v_s + i, a.v + ((size_t)(row0 + t0 + tt) * H + h) * dv + col0 + c);
    }
    if (DELTA || TOKEN_DECAY)
      for (int i = tid; i < nt; i += THREADS) cp_async4(b_s + i, a.beta + (size_t)(row0 + t0 + i) * H + h);
  };
  const float decay = (CHANNEL || TOKEN_DECAY) ? 1.f : a.head_decay[h];
  load(0, 0);
  cp_async_commit();
  for (int t0 = 0, it = 0; t0 < n_tok; t0 += TS, ++it) {
    const int st = it & 1;
    if (t0 + TS < n_tok) {
      load(t0 + TS, st ^ 1);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const int nt = min(TS, n_tok - t0);
    const float* q_s = stage + st * per_stage;
    const float* k_s = q_s + TS * DP;
    const float* g_s = k_s + TS * DP;
    const float* v_s = stage + st * per_stage + TS * DP * (CHANNEL ? 3 : 2);
    const float* b_s = v_s + TS * CPB;
    // Without the delta rule a token's output is off the chain from token to token (only S is carried), so four or eight
    // tokens go through the update one after another and their outputs' sums over the lanes of a column are then formed
    // side by side: independent chains of shuffles instead of one a token.
    constexpr int TU = (!DELTA && R >= 8) ? (ROWS <= 4 ? 8 : 4) : 1;
    for (int tt = 0; tt < nt; tt += TU) {
      float o_part[TU];
#pragma unroll
      for (int j = 0; j < TU; ++j) {
        o_part[j] = 0.f;
        const int tj = tt + j;
        if (TU > 1 && tj >= nt) continue;  // the same for every thread of the block
        // this lane's rows of q, k and g as 16-byte words (ROWS and DP are multiples of 4)
        float qv[ROWS], kv[ROWS], gv[CHANNEL ? ROWS : 1];
#pragma unroll
        for (int i = 0; i < ROWS; i += 4) {
          *reinterpret_cast<float4*>(qv + i) = *reinterpret_cast<const float4*>(q_s + tj * DP + r * ROWS + i);
          *reinterpret_cast<float4*>(kv + i) = *reinterpret_cast<const float4*>(k_s + tj * DP + r * ROWS + i);
          if (CHANNEL) *reinterpret_cast<float4*>(gv + i) = *reinterpret_cast<const float4*>(g_s + tj * DP + r * ROWS + i);
        }
        float u = live ? v_s[tj * CPB + warp * CPW + cw] : 0.f;
        if (DELTA) {
          float p4[4] = {0.f, 0.f, 0.f, 0.f};  // four sums side by side: the chain of additions is a quarter as long
#pragma unroll
          for (int i = 0; i < ROWS; ++i) {
            s[i] *= gv[i];
            p4[i & 3] = fmaf(s[i], kv[i], p4[i & 3]);
          }
          float part = (p4[0] + p4[1]) + (p4[2] + p4[3]);
#pragma unroll
          for (int o = CPW; o < 32; o <<= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
          u = b_s[tj] * (u - part);
        }
        float o4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int i = 0; i < ROWS; ++i) {
          if (MODE == 1) s[i] = fmaf(kv[i], u, s[i]);
          else if (MODE == 2) s[i] = fmaf(gv[i], s[i], kv[i] * u);
          else if (MODE == 3) s[i] = fmaf(b_s[tj], s[i], kv[i] * u);
          else s[i] = fmaf(decay, s[i], kv[i] * u);
          o4[i & 3] = fmaf(s[i], qv[i], o4[i & 3]);
        }
        o_part[j] = (o4[0] + o4[1]) + (o4[2] + o4[3]);
      }
#pragma unroll
      for (int o = CPW; o < 32; o <<= 1)
#pragma unroll
        for (int j = 0; j < TU; ++j) o_part[j] += __shfl_xor_sync(0xffffffffu, o_part[j], o);
#pragma unroll
      for (int j = 0; j < TU; ++j)
        if (live && r == 0 && tt + j < nt) a.out[((size_t)(row0 + t0 + tt + j) * H + h) * dv + col] = o_part[j];
    }
    __syncthreads();  // this stage is loaded again two rounds on
  }
  if (live) {
#pragma unroll
    for (int i = 0; i < ROWS; ++i) {
      const int row = r * ROWS + i;
      if (row < d) S[(size_t)row * dv + col] = s[i];
    }
  }
}

template <int ROWS, int R, int MODE, int THREADS = SCAN_THREADS>
int launch_scan(const ScanArgs& args, int n_seqs, cudaStream_t stream) {
  ScanArgs a = args;
  constexpr int DP = ROWS * R, CPB = (32 / R) * (THREADS / 32);
  a.tok_stage = DP <= 128 ? 16 : (DP <= 256 ? 8 : (DP <= 512 ? 4 : 2));
  const size_t smem = (size_t)2 * ((a.tok_stage * DP * ((MODE == 1 || MODE == 2) ? 3 : 2) + a.tok_stage * CPB + a.tok_stage + 3) & ~3) * sizeof(float);
  const dim3 grid((a.dv + CPB - 1) / CPB, a.n_heads, n_seqs);
  if (smem > 48 * 1024) {
    cudaError_t err = cudaFuncSetAttribute(state_scan_kernel<ROWS, R, MODE, THREADS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (err != cudaSuccess) {
      mll_set_error("state scan: cannot reserve %zu bytes of shared memory: %s", smem, cudaGetErrorString(err));
      return (int)err;
    }
  }
  MLL_LAUNCH((state_scan_kernel<ROWS, R, MODE, THREADS>), grid, THREADS, smem, stream, a);
  MLL_LAUNCH_CHECK();
  return 0;
}

// How a column of S is spread over lanes.  With enough columns to fill the device (a decode step of a batch) a
// thread holds a whole column (keys up to 64; two lanes up to 128, four up to 256: 64 rows are what a thread's
// registers hold): a warp then reads and writes 128, 64 or 32 consecutive bytes of a row of the state.  Measured
// on 128 sequences of 16 heads of 128 x 128 (134 MB of state in and out): 64 rows a lane 112 us (2.4 TB/s); 32
// rows a lane and four lanes a column, with twice the resident blocks, 142 us.  That layout starts at 256 columns a
// multiprocessor (64 sequences of 8 heads of 128 value columns: 51 us with eight lanes a column, whose 16-byte pieces
// of a row use half of every sector, 29 us with two).  Otherwise (a prompt of one or a few sequences) eight lanes
// share a column, so that eight times as many threads work on the chain from token to token - or, with very few
// columns, a whole warp (below).
template <int MODE>
int dispatch_scan(const ScanArgs& a, int n_seqs, cudaStream_t stream) {
  const int d = a.d;
  const bool many = (long long)n_seqs * a.n_heads * a.dv >= (long long)mll_sm_count() * 256;
  if (many && d <= 32) return launch_scan<32, 1, MODE>(a, n_seqs, stream);
  if (many && d <= 64) return launch_scan<64, 1, MODE>(a, n_seqs, stream);
  if (many && d <= 128) return launch_scan<64, 2, MODE>(a, n_seqs, stream);
  if (many && d <= 256) return launch_scan<64, 4, MODE>(a, n_seqs, stream);
  // So few columns that eight lanes a column leave a multiprocessor with two or three warps (one prompt of a model a
  // few thousand wide), each of which waits out the latency of its own instructions: a whole warp a column (half a
  // warp for keys up to 64) - four rows a lane, a quarter of the arithmetic in every step of the chain from token to
  // token - and eight warps a block, so that a block still stages a token's q, k and g once for eight columns.
  // Not for the delta rule, whose sum over a column's lanes lies on the chain.
  const bool few = MODE != 1 && (long long)n_seqs * a.n_heads * a.dv < (long long)mll_sm_count() * 16;
  if (few && d > 32 && d <= 64) return launch_scan<4, 16, MODE, 256>(a, n_seqs, stream);
  if (few && d > 64 && d <= 128) return launch_scan<4, 32, MODE, 256>(a, n_seqs, stream);
  if (few && d > 128 && d <= 256) return launch_scan<8, 32, MODE, 256>(a, n_seqs, stream);
  if (d <= 32) return launch_scan<4, 8, MODE>(a, n_seqs, stream);
  if (d <= 64) return launch_scan<8, 8, MODE>(a, n_seqs, stream);
  if (d <= 128) return launch_scan<16, 8, MODE>(a, n_seqs, stream);
  if (d <= 256) return launch_scan<32, 8, MODE>(a, n_seqs, stream);
  return launch_scan<32, 32, MODE>(a, n_seqs, stream);
}

// ---------------------------------------------------------------------------------------------- //
// grid (tokens, ceil(H / 4)), one warp per (token, head):
//   out[t, h, :] = o / sqrt(mean(o^2) + eps) * weight * act(gate[t, h, :])      act: 0 silu, 1 sigmoid
template <typename T, typename GateT>
__global__ void __launch_bounds__(128) head_norm_gate_kernel(const float* __restrict__ o, const float* __restrict__ weight,
                                                             const GateT* __restrict__ gate, int gate_ld,
                                                             T* __restrict__ out, int n_heads, int dv, float eps,
                                                             int act) {
  const int t = blockIdx.x;
  const int h = blockIdx.y * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (h >= n_heads) return;
  const float* row = o + ((size_t)t * n_heads + h) * dv;
  float ss = 0.f;
  for (int e = lane; e < dv; e += 32) ss += row[e] * row[e];
  ss = warp_sum(ss);
  const float f = 1.f / sqrtf(ss / (float)dv + eps);
  const GateT* grow = gate + (size_t)t * gate_ld + (size_t)h * dv;
  T* dst = out + ((size_t)t * n_heads + h) * dv;
  for (int e = lane; e < dv; e += 32) {
    const float z = to_float(grow[e]);
    const float gv = act == 0 ? silu_f(z) : sigmoid_f(z);
    dst[e] = from_float<T>(row[e] * f * (weight ? weight[e] : 1.f) * gv);
  }
}

// grid (tokens, parts), 256 threads: a row of o [H dv] in `parts` equal pieces, each normalised by its own root mean
// square after the skip and the gate:   y = (o + skip[h] xs) * silu(z);   out = y / sqrt(mean_part(y^2) + eps) * weight
template <typename T, typename GateT>
__global__ void __launch_bounds__(256) gated_group_norm_kernel(const float* __restrict__ o, const float* __restrict__ xs,
                                                               const float* __restrict__ skip,
                                                               const GateT* __restrict__ gate, int gate_ld,
                                                               const float* __restrict__ weight, T* __restrict__ out,
                                                               int width, int dv, int parts, float eps) {
  __shared__ float scratch[32];
  const int t = blockIdx.x, part = blockIdx.y;
  const int n = width / parts, c0 = part * n;
  const float* orow = o + (size_t)t * width + c0;
  const float* xrow = xs ? xs + (size_t)t * width + c0 : nullptr;
  const GateT* grow = gate + (size_t)t * gate_ld + c0;
  // a part of up to 8 x 256 columns stays in registers between the sum and the scaling: one pass over the inputs
  constexpr int KEEP = 8;
  const bool kept = n <= KEEP * 256;
  float held[KEEP];
  float ss = 0.f;
  if (kept) {
#pragma unroll
    for (int i = 0; i < KEEP; ++i) {
      const int e = threadIdx.x + i * 256;
      float y = 0.f;
      if (e < n) {
        y = orow[e];
        if (xrow) y = fmaf(skip[(c0 + e) / dv], xrow[e], y);
        y *= silu_f(to_float(grow[e]));
      }
      held[i] = y;
      ss += y * y;
    }
  } else {
    for (int e = threadIdx.x; e < n; e += blockDim.x) {
      float y = orow[e];
      if (xrow) y = fmaf(skip[(c0 + e) / dv], xrow[e], y);
      y *= silu_f(to_float(grow[e]));
      ss += y * y;
    }
  }
  ss = block_sum(ss, scratch);
  const float f = 1.f / sqrtf(ss / (float)n + eps);
  T* dst = out + (size_t)t * width + c0;
  if (kept) {
#pragma unroll
    for (int i = 0; i < KEEP; ++i) {
      const int e = threadIdx.x + i * 256;
      if (e < n) dst[e] = from_float<T>(held[i] * f * weight[c0 + e]);
    }
    return;
  }
  for (int e = threadIdx.x; e < n; e += blockDim.x) {
    float y = orow[e];
    if (xrow) y = fmaf(skip[(c0 + e) / dv], xrow[e], y);
    y *= silu_f(to_float(grow[e]));
    dst[e] = from_float<T>(y * f * weight[c0 + e]);
  }
}

}  // namespace mll

MLL_API int mll_ssd_prepare(const void* proj, const float* conv_w, const float* conv_b, const float* conv_state,
                            const float* a_log, const float* dt_bias, const int* tok_seq, const int* seq_slot,
                            const int* seq_qstart, float* q, float* k, float* u, float* xs, float* decay, int dtype,
                            int n_tokens, int ld, int n_heads, int n_groups, int d, int dv, int taps,
                            cudaStream_t stream) {
  MLL_REQUIRE(n_tokens >= 0 && n_heads > 0 && n_groups > 0 && n_heads % n_groups == 0, "ssd prepare: bad head counts");
  MLL_REQUIRE(d > 0 && dv > 0 && taps >= 1, "ssd prepare: bad sizes");
  MLL_REQUIRE(ld >= 2 * n_heads * dv + 2 * n_groups * d + n_heads, "ssd prepare: row stride %d too short", ld);
  MLL_REQUIRE(n_heads <= 8192, "ssd prepare: %d heads (at most 8192)", n_heads);
  if (n_tokens == 0) return 0;
  mll::SsdPrepArgs a{proj, conv_w, conv_b, conv_state, a_log, dt_bias, tok_seq, seq_slot, seq_qstart, q, k, u, xs, decay,
                     ld, n_heads, n_groups, d, dv, taps};
  const size_t smem = (size_t)n_heads * sizeof(float);
  const int channels = n_heads * dv + 2 * n_groups * d;
  // a prompt fills the device with a block a token, which walks its channels (2,048 tokens of 6,144 channels: 115 us
  // against 176 us in pieces); a step of few tokens is cut into pieces of 256 channels (64 tokens: 41 -> 20 us)
  const int per_block = n_tokens >= 4 * mll_sm_count() ? channels : 256;
  const dim3 grid(n_tokens, (channels + per_block - 1) / per_block);
  MLL_REQUIRE(grid.y <= 65535, "ssd prepare: too many channels for one launch");
  if (dtype == MLL_F32)
    MLL_LAUNCH((mll::ssd_prepare_kernel<float>), grid, 256, smem, stream, a, per_block);
  else if (dtype == MLL_BF16)
    MLL_LAUNCH((mll::ssd_prepare_kernel<__nv_bfloat16>), grid, 256, smem, stream, a, per_block);
  else
    MLL_REQUIRE(false, "ssd prepare: unknown dtype %d", dtype);
  MLL_LAUNCH_CHECK();
  return 0;
}

MLL_API int mll_gated_group_norm(const float* o, const float* xs, const float* skip, const void* gate, int gate_dtype,
                                 int gate_ld, const float* weight, void* out, int out_dtype, int n_tokens, int width,
                                 int dv, int parts, float eps, cudaStream_t stream) {
  MLL_REQUIRE(n_tokens >= 0 && width > 0 && dv > 0 && parts > 0 && width % parts == 0 && gate_ld >= width,
              "gated group norm: bad sizes width=%d parts=%d", width, parts);
  MLL_REQUIRE((xs == nullptr) == (skip == nullptr), "gated group norm: a skip needs its input and its factors");
  MLL_REQUIRE(parts <= 65535, "gated group norm: too many parts for one launch");
  if (n_tokens == 0) return 0;
  const dim3 grid(n_tokens, parts);
#define MLL_GGN(T, GT)                                                                                             \
  MLL_LAUNCH((mll::gated_group_norm_kernel<T, GT>), grid, 256, 0, stream, o, xs, skip, (const GT*)gate, gate_ld, \
             weight, (T*)out, width, dv, parts, eps)
  if (out_dtype == MLL_F32 && gate_dtype == MLL_F32) MLL_GGN(float, float);
  else if (out_dtype == MLL_BF16 && gate_dtype == MLL_BF16) MLL_GGN(__nv_bfloat16, __nv_bfloat16);
  else MLL_REQUIRE(false, "gated group norm: dtypes %d / %d", out_dtype, gate_dtype);
#undef MLL_GGN
  MLL_LAUNCH_CHECK();
  return 0;
}

MLL_API int mll_retention_prepare(const void* proj, const float* cos_table, const float* sin_table, const int* tok_pos,
                                  float* q, float* k, float* v, int dtype, int n_tokens, int ld, int n_heads, int d,
                                  int dv, int rot, int interleaved, float k_scale, cudaStream_t stream) {
  MLL_REQUIRE(n_tokens >= 0 && n_heads > 0 && d > 0 && dv > 0, "retention prepare: bad sizes");
  MLL_REQUIRE(rot >= 0 && rot <= d && rot % 2 == 0, "retention prepare: %d rotated dimensions of %d", rot, d);
  MLL_REQUIRE(ld >= n_heads * (2 * d + dv), "retention prepare: row stride %d too short", ld);
  if (n_tokens == 0) return 0;
  mll::RetPrepArgs a{proj, rot > 0 ? cos_table : nullptr, sin_table, tok_pos, q, k, v, ld, n_heads, d, dv, rot,
                     interleaved, k_scale};
  if (dtype == MLL_F32)
    MLL_LAUNCH((mll::retention_prepare_kernel<float>), n_tokens, 256, 0, stream, a);
  else if (dtype == MLL_BF16)
    MLL_LAUNCH((mll::retention_prepare_kernel<__nv_bfloat16>), n_tokens, 256, 0, stream, a);
  else
    MLL_REQUIRE(false, "retention prepare: unknown dtype %d", dtype);
  MLL_LAUNCH_CHECK();
  return 0;
}

MLL_API int mll_delta_prepare(const void* proj, const float* rate, const float* conv_w, const float* conv_state,
                              const float* a_log, const float* dt_bias, const int* tok_seq, const int* seq_slot,
                              const int* seq_qstart, float* q, float* k, float* v, float* g, float* beta, int dtype,
                              int n_tokens, int ld, int rate_ld, int n_heads, int n_kv_heads, int d, int dv, int taps,
                              float unit_eps, cudaStream_t stream) {
  MLL_REQUIRE(n_tokens >= 0 && n_heads > 0 && n_kv_heads > 0 && n_heads % n_kv_heads == 0, "delta prepare: bad head counts");
  MLL_REQUIRE(d > 0 && dv > 0 && taps >= 1, "delta prepare: bad sizes");
  const int C = 2 * n_kv_heads * d + n_heads * dv;
  MLL_REQUIRE(ld >= C + n_heads && rate_ld >= n_heads * d, "delta prepare: row strides %d / %d too short", ld, rate_ld);
  MLL_REQUIRE(d <= 2048 && dv <= 2048 && 2 * n_kv_heads + n_heads <= 65535, "delta prepare: heads too large or too many");
  if (n_tokens == 0) return 0;
  mll::DeltaPrepArgs a{proj, rate, conv_w, conv_state, a_log, dt_bias, tok_seq, seq_slot, seq_qstart, q, k, v, g, beta,
                       ld, rate_ld, n_heads, n_kv_heads, d, dv, taps, unit_eps};
  const size_t smem = (size_t)4 * (d > dv ? d : dv) * sizeof(float);
  const dim3 grid((n_tokens + 3) / 4, 2 * n_kv_heads + n_heads);
  if (dtype == MLL_F32)
    MLL_LAUNCH((mll::delta_prepare_kernel<float>), grid, 128, smem, stream, a, n_tokens);
  else if (dtype == MLL_BF16)
    MLL_LAUNCH((mll::delta_prepare_kernel<__nv_bfloat16>), grid, 128, smem, stream, a, n_tokens);
  else
    MLL_REQUIRE(false, "delta prepare: unknown dtype %d", dtype);
  MLL_LAUNCH_CHECK();
  return 0;
}

MLL_API int mll_channel_decay_prepare(const void* proj, const float* rate, const float* bias, float* q, float* k, float* v,
                                      float* g, int dtype, int n_tokens, int ld, int rate_ld, int n_heads, int d, int dv,
                                      float q_scale, float tau, cudaStream_t stream) {
  MLL_REQUIRE(n_tokens >= 0 && n_heads > 0 && d > 0 && dv > 0, "channel decay prepare: bad sizes");
  MLL_REQUIRE(ld >= n_heads * (2 * d + dv) && rate_ld >= n_heads * d, "channel decay prepare: row strides %d / %d too short", ld, rate_ld);
  MLL_REQUIRE(tau > 0.f, "channel decay prepare: tau must be positive");
  if (n_tokens == 0) return 0;
  mll::ChannelDecayArgs a{proj, rate, bias, q, k, v, g, ld, rate_ld, n_heads, d, dv, q_scale, 1.f / tau};
  if (dtype == MLL_F32)
    MLL_LAUNCH((mll::channel_decay_prepare_kernel<float>), n_tokens, 256, 0, stream, a);
  else if (dtype == MLL_BF16)
    MLL_LAUNCH((mll::channel_decay_prepare_kernel<__nv_bfloat16>), n_tokens, 256, 0, stream, a);
  else
    MLL_REQUIRE(false, "channel decay prepare: unknown dtype %d", dtype);
  MLL_LAUNCH_CHECK();
  return 0;
}

MLL_API int mll_conv_state_update(const void* proj, int dtype, int col0, int ld, float* conv_state, const int* seq_slot,
                                  const int* seq_qstart, const int* seq_qlen, int n_seqs, int channels, int taps,
                                  cudaStream_t stream) {
  MLL_REQUIRE(n_seqs >= 0 && channels > 0 && taps >= 1 && col0 >= 0 && ld >= col0 + channels, "conv state update: bad sizes");
  if (n_seqs == 0 || taps == 1) return 0;
  MLL_REQUIRE(n_seqs <= 65535, "conv state update: too many sequences for one launch");
  const dim3 grid((channels + 127) / 128, n_seqs);
  if (dtype == MLL_F32)
    MLL_LAUNCH((mll::conv_state_update_kernel<float>), grid, 128, 0, stream, (const float*)proj, col0, ld,
               conv_state, seq_slot, seq_qstart, seq_qlen, channels, taps);
  else if (dtype == MLL_BF16)
    MLL_LAUNCH((mll::conv_state_update_kernel<__nv_bfloat16>), grid, 128, 0, stream, (const __nv_bfloat16*)proj,
               col0, ld, conv_state, seq_slot, seq_qstart, seq_qlen, channels, taps);
  else
    MLL_REQUIRE(false, "conv state update: unknown dtype %d", dtype);
  MLL_LAUNCH_CHECK();
  return 0;
}

// mode 1: the gated delta rule (g, beta given); 2: a decay per key channel without the delta rule (g given);
// 0: one decay per head (head_decay given); 3: one decay per token and head (beta [T, H] holds it).
MLL_API int mll_state_scan(const float* q, const float* k, const float* v, const float* g, const float* beta,
                           const float* head_decay, float* state, float* out, const int* seq_slot,
                           const int* seq_qstart, const int* seq_qlen, int n_seqs, int n_heads, int n_kv_heads, int d,
                           int dv, int mode, cudaStream_t stream) {
  MLL_REQUIRE(n_seqs >= 0 && n_heads > 0 && n_kv_heads > 0 && n_heads % n_kv_heads == 0, "state scan: bad head counts");
  MLL_REQUIRE(d > 0 && d <= 1024 && dv > 0, "state scan: head sizes %d / %d (keys at most 1024)", d, dv);
  MLL_REQUIRE(n_heads <= 65535 && n_seqs <= 65535, "state scan: too many heads or sequences for one launch");
  MLL_REQUIRE(mode >= 0 && mode <= 3, "state scan: unknown mode %d", mode);
  MLL_REQUIRE(mode == 1 ? (g && beta) : (mode == 2 ? g != nullptr : (mode == 3 ? beta != nullptr : head_decay != nullptr)),
              "state scan: the decay's inputs are missing");
  if (n_seqs == 0) return 0;
  mll::ScanArgs a{q, k, v, g, beta, head_decay, state, out, seq_slot, seq_qstart, seq_qlen, n_heads, n_kv_heads, d, dv, 0};
  if (mode == 1) return mll::dispatch_scan<1>(a, n_seqs, stream);
  if (mode == 2) return mll::dispatch_scan<2>(a, n_seqs, stream);
  if (mode == 3) return mll::dispatch_scan<3>(a, n_seqs, stream);
  return mll::dispatch_scan<0>(a, n_seqs, stream);
}

MLL_API int mll_head_norm_gate(const float* o, const float* weight, const void* gate, int gate_dtype, int gate_ld,
                               void* out, int out_dtype, int n_tokens, int n_heads, int dv, float eps, int act,
                               cudaStream_t stream) {
  MLL_REQUIRE(n_tokens >= 0 && n_heads > 0 && dv > 0 && gate_ld >= n_heads * dv, "head norm gate: bad sizes");
  MLL_REQUIRE(act == 0 || act == 1, "head norm gate: unknown activation %d", act);
  if (n_tokens == 0) return 0;
  const dim3 grid(n_tokens, (n_heads + 3) / 4);
  MLL_REQUIRE(grid.y <= 65535, "head norm gate: too many heads for one launch");
#define MLL_HNG(T, GT)                                                                                          \
  MLL_LAUNCH((mll::head_norm_gate_kernel<T, GT>), grid, 128, 0, stream, o, weight, (const GT*)gate, gate_ld, \
             (T*)out, n_heads, dv, eps, act)
  if (out_dtype == MLL_F32 && gate_dtype == MLL_F32) MLL_HNG(float, float);
  else if (out_dtype == MLL_BF16 && gate_dtype == MLL_BF16) MLL_HNG(__nv_bfloat16, __nv_bfloat16);
  else if (out_dtype == MLL_BF16 && gate_dtype == MLL_F32) MLL_HNG(__nv_bfloat16, float);
  else MLL_REQUIRE(false, "head norm gate: dtypes %d / %d", out_dtype, gate_dtype);
#undef MLL_HNG
  MLL_LAUNCH_CHECK();
  return 0;
}
