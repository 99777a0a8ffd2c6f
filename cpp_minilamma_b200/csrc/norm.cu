// RMSNorm fused with the residual add, and the gathered variant for the final norm.
//
//   x[t, :] += delta[t, :]            (float32 residual stream, updated in place)
//   out[t, i] = x[t, i] * w[i] / sqrt(mean_j(x[t, j]^2) + eps)
//
// The formula is the reference's (src/ops.cc:95-110; eps inside the root).  Its GPU
// version sums squares with float atomics (src/cuda_ops.cu:151-164), which is not
// reproducible; here every row is reduced by one block with a fixed tree, in float32.
#include "common.cuh"

namespace mll {

// What happens to the delta on its way into the stream: delta = scale1 * delta (+ scale2 * delta2), and with a
// weight the delta is normalised by its own root mean square first: x += delta / sqrt(mean(delta^2) + eps) * weight
// (a block whose sub-layers end in a norm of their own).
struct DeltaNorm {
  const float* weight;  // [width] or null: the delta is added as it is
  float eps, scale1, scale2;
};

// One block per output row.  The row (after the add) is kept in shared memory between
// the two passes.  `rows` (optional) selects which rows of x are normalised: output row
// r reads x row rows[r]; the residual add is then not written back to x.
template <typename DeltaT, typename OutT>
__global__ void add_rmsnorm_kernel(float* __restrict__ x, const DeltaT* __restrict__ delta,
                                   const DeltaT* __restrict__ delta2,
                                   const float* __restrict__ weight, OutT* __restrict__ out,
                                   const int* __restrict__ rows, int width, float eps, DeltaNorm dn) {
  extern __shared__ float row_buf[];
  __shared__ float scratch[32];
  const int r = blockIdx.x;
  const int src = rows ? rows[r] : r;
  float* xr = x + (size_t)src * width;
  const DeltaT* dr = delta ? delta + (size_t)src * width : nullptr;
  const DeltaT* dr2 = delta2 ? delta2 + (size_t)src * width : nullptr;
  float fd = 1.f;
  if (dr && dn.weight) {  // the delta passes a norm of its own before it joins the stream
    float sd = 0.f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
      const float d = dr2 ? dn.scale1 * to_float(dr[i]) + dn.scale2 * to_float(dr2[i]) : dn.scale1 * to_float(dr[i]);
      sd += d * d;
    }
    fd = 1.f / sqrtf(block_sum(sd, scratch) / (float)width + dn.eps);
  }
  float ss = 0.f;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    float v = xr[i];
    if (dr) {
      const float d = dr2 ? dn.scale1 * to_float(dr[i]) + dn.scale2 * to_float(dr2[i]) : dn.scale1 * to_float(dr[i]);
      v += dn.weight ? d * fd * dn.weight[i] : d;
      if (!rows) xr[i] = v;
    }
    row_buf[i] = v;
    ss += v * v;
  }
  ss = block_sum(ss, scratch);
  const float scale = 1.f / sqrtf(ss / (float)width + eps);
  OutT* o = out + (size_t)r * width;
  for (int i = threadIdx.x; i < width; i += blockDim.x)
    o[i] = from_float<OutT>(row_buf[i] * scale * weight[i]);
}

// Rows whose width is a multiple of 4 and at most 4 * NV * blockDim: every thread keeps
// its share of the row in registers and issues all its loads before the first use, so the
// kernel costs one memory latency instead of one per loop trip (decode has very few rows).
template <typename T>
__device__ __forceinline__ float4 load4(const T* p);
template <>
__device__ __forceinline__ float4 load4<float>(const float* p) {
  return *reinterpret_cast<const float4*>(p);
}
template <>
__device__ __forceinline__ float4 load4<__nv_bfloat16>(const __nv_bfloat16* p) {
  const uint2 raw = *reinterpret_cast<const uint2*>(p);
  const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
  const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
  return make_float4(a.x, a.y, b.x, b.y);
}
__device__ __forceinline__ void store4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void store4(__nv_bfloat16* p, float4 v) {
  __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
  uint2 raw;
  raw.x = *reinterpret_cast<unsigned*>(&lo);
  raw.y = *reinterpret_cast<unsigned*>(&hi);
  *reinterpret_cast<uint2*>(p) = raw;
}

template <typename DeltaT, typename OutT, int NV>
__global__ void __launch_bounds__(256)
add_rmsnorm_vec_kernel(float* __restrict__ x, const DeltaT* __restrict__ delta,
                       const DeltaT* __restrict__ delta2,
                       const float* __restrict__ weight, OutT* __restrict__ out,
                       const int* __restrict__ rows, int width, float eps, DeltaNorm dn) {
  __shared__ float scratch[32];
  const int r = blockIdx.x;
  const int src = rows ? rows[r] : r;
  float* xr = x + (size_t)src * width;
  const DeltaT* dr = delta ? delta + (size_t)src * width : nullptr;
  const int groups = width >> 2;
  float4 v[NV], w[NV];
#pragma unroll
  for (int k = 0; k < NV; ++k) {
    const int g = threadIdx.x + k * 256;
    if (g < groups) {
      v[k] = load4<float>(xr + 4 * g);
      w[k] = load4<float>(weight + 4 * g);
    }
  }
  if (dr) {
    float4 dl[NV];
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      const int g = threadIdx.x + k * 256;
      if (g < groups) {
        dl[k] = load4<DeltaT>(dr + 4 * g);
        if (dn.scale1 != 1.f) { dl[k].x *= dn.scale1; dl[k].y *= dn.scale1; dl[k].z *= dn.scale1; dl[k].w *= dn.scale1; }
        if (delta2) {  // the outputs of two parts that read the same norm: their sum first, then the stream
          const float4 d2 = load4<DeltaT>(delta2 + (size_t)src * width + 4 * g);
          dl[k].x = fmaf(dn.scale2, d2.x, dl[k].x); dl[k].y = fmaf(dn.scale2, d2.y, dl[k].y);
          dl[k].z = fmaf(dn.scale2, d2.z, dl[k].z); dl[k].w = fmaf(dn.scale2, d2.w, dl[k].w);
        }
      }
    }
    if (dn.weight) {  // the delta's own norm (uniform over the block: every thread takes part in the sum)
      float sd = 0.f;
#pragma unroll
      for (int k = 0; k < NV; ++k) {
        const int g = threadIdx.x + k * 256;
        if (g < groups) sd += dl[k].x * dl[k].x + dl[k].y * dl[k].y + dl[k].z * dl[k].z + dl[k].w * dl[k].w;
      }
      const float fd = 1.f / sqrtf(block_sum(sd, scratch) / (float)width + dn.eps);
      __syncthreads();  // scratch is used again below
#pragma unroll
      for (int k = 0; k < NV; ++k) {
        const int g = threadIdx.x + k * 256;
        if (g < groups) {
          const float4 dw = load4<float>(dn.weight + 4 * g);
          dl[k].x *= fd * dw.x; dl[k].y *= fd * dw.y; dl[k].z *= fd * dw.z; dl[k].w *= fd * dw.w;
        }
      }
    }
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      const int g = threadIdx.x + k * 256;
      if (g < groups) {
        v[k].x += dl[k].x; v[k].y += dl[k].y; v[k].z += dl[k].z; v[k].w += dl[k].w;
        if (!rows) store4(xr + 4 * g, v[k]);
      }
    }
  }
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < NV; ++k) {
    const int g = threadIdx.x + k * 256;
    if (g < groups) ss += v[k].x * v[k].x + v[k].y * v[k].y + v[k].z * v[k].z + v[k].w * v[k].w;
  }
  ss = block_sum(ss, scratch);
  const float scale = 1.f / sqrtf(ss / (float)width + eps);
  OutT* o = out + (size_t)r * width;
#pragma unroll
  for (int k = 0; k < NV; ++k) {
    const int g = threadIdx.x + k * 256;
    if (g < groups)
      store4(o + 4 * g, make_float4(v[k].x * scale * w[k].x, v[k].y * scale * w[k].y, v[k].z * scale * w[k].z,
                                    v[k].w * scale * w[k].w));
  }
}

template <typename DeltaT, typename OutT>
int launch_add_rmsnorm(float* x, const void* delta, const void* delta2, const float* weight, void* out,
                       const int* rows, int n_rows, int width, float eps, DeltaNorm dn, cudaStream_t stream) {
  const bool aligned = width % 4 == 0 && ((uintptr_t)x % 16 == 0) && ((uintptr_t)weight % 16 == 0) &&
                       ((uintptr_t)out % 16 == 0) && (!delta || (uintptr_t)delta % 8 == 0) &&
                       (!delta2 || (uintptr_t)delta2 % 8 == 0) && (!dn.weight || (uintptr_t)dn.weight % 16 == 0);
  if (aligned && width <= 4 * 256 * 8) {
    const int groups = width / 4;
    if (groups <= 256 * 2)
      MLL_LAUNCH((add_rmsnorm_vec_kernel<DeltaT, OutT, 2>), n_rows, 256, 0, stream, x, (const DeltaT*)delta,
                 (const DeltaT*)delta2, weight, (OutT*)out, rows, width, eps, dn);
    else if (groups <= 256 * 4)
      MLL_LAUNCH((add_rmsnorm_vec_kernel<DeltaT, OutT, 4>), n_rows, 256, 0, stream, x, (const DeltaT*)delta,
                 (const DeltaT*)delta2, weight, (OutT*)out, rows, width, eps, dn);
    else
      MLL_LAUNCH((add_rmsnorm_vec_kernel<DeltaT, OutT, 8>), n_rows, 256, 0, stream, x, (const DeltaT*)delta,
                 (const DeltaT*)delta2, weight, (OutT*)out, rows, width, eps, dn);
    MLL_LAUNCH_CHECK();
    return 0;
  }
  const int threads = width >= 2048 ? 512 : (width >= 512 ? 256 : 128);
  const size_t smem = (size_t)width * sizeof(float);
  auto kernel = add_rmsnorm_kernel<DeltaT, OutT>;
  if (smem > 48 * 1024) {
    cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (err != cudaSuccess) {
      mll_set_error("rmsnorm: cannot reserve %zu bytes of shared memory: %s", smem, cudaGetErrorString(err));
      return (int)err;
    }
  }
  MLL_LAUNCH((kernel), n_rows, threads, smem, stream, x, (const DeltaT*)delta, (const DeltaT*)delta2, weight,
             (OutT*)out, rows, width, eps, dn);
  MLL_LAUNCH_CHECK();
  return 0;
}

// Layer norm with weight and bias, fused with the residual add like the kernel above:
//   x[t, :] += delta[t, :];   out[t, i] = (x[t, i] - mean) / sqrt(var + eps) * w[i] + b[i]
// with var the mean of the squared deviations from the mean (two passes over the row, which stays in shared
// memory; float32 throughout).  One block per output row; `rows` gathers as above.
template <typename DeltaT, typename OutT>
__global__ void add_layernorm_kernel(float* __restrict__ x, const DeltaT* __restrict__ delta,
                                     const float* __restrict__ weight, const float* __restrict__ bias,
                                     OutT* __restrict__ out, const int* __restrict__ rows, int width, float eps) {
  extern __shared__ float row_buf[];
  __shared__ float scratch[32];
  const int r = blockIdx.x;
  const int src = rows ? rows[r] : r;
  float* xr = x + (size_t)src * width;
  const DeltaT* dr = delta ? delta + (size_t)src * width : nullptr;
  float sum = 0.f;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    float v = xr[i];
    if (dr) {
      v += to_float(dr[i]);
      if (!rows) xr[i] = v;
    }
    row_buf[i] = v;
    sum += v;
  }
  const float mean = block_sum(sum, scratch) / (float)width;
  float dev = 0.f;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    const float c = row_buf[i] - mean;
    dev += c * c;
  }
  const float scale = 1.f / sqrtf(block_sum(dev, scratch) / (float)width + eps);
  OutT* o = out + (size_t)r * width;
  for (int i = threadIdx.x; i < width; i += blockDim.x)
    o[i] = from_float<OutT>((row_buf[i] - mean) * scale * weight[i] + (bias ? bias[i] : 0.f));
}

// The same with the row in registers (widths that are multiples of 4, up to 4 * NV * 256): every thread issues all its
// loads before the first use, and the two passes (mean, then squared deviations) run over registers.
template <typename DeltaT, typename OutT, int NV>
__global__ void __launch_bounds__(256)
add_layernorm_vec_kernel(float* __restrict__ x, const DeltaT* __restrict__ delta, const float* __restrict__ weight,
                         const float* __restrict__ bias, OutT* __restrict__ out, const int* __restrict__ rows, int width,
                         float eps) {
  __shared__ float scratch[32];
  const int r = blockIdx.x;
  const int src = rows ? rows[r] : r;
  float* xr = x + (size_t)src * width;
  const DeltaT* dr = delta ? delta + (size_t)src * width : nullptr;
  const int groups = width >> 2;
  float4 v[NV];
#pragma unroll
  for (int k = 0; k < NV; ++k) {
    const int g = threadIdx.x + k * 256;
    v[k] = g < groups ? load4<float>(xr + 4 * g) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  if (dr) {
    float4 dl[NV];
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      const int g = threadIdx.x + k * 256;
      if (g < groups) dl[k] = load4<DeltaT>(dr + 4 * g);
    }
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      const int g = threadIdx.x + k * 256;
      if (g < groups) {
        v[k].x += dl[k].x; v[k].y += dl[k].y; v[k].z += dl[k].z; v[k].w += dl[k].w;
        if (!rows) store4(xr + 4 * g, v[k]);
      }
    }
  }
  float sum = 0.f;
#pragma unroll
  for (int k = 0; k < NV; ++k) sum += (v[k].x + v[k].y) + (v[k].z + v[k].w);  // groups past the row hold zeros
  const float mean = block_sum(sum, scratch) / (float)width;
  float dev = 0.f;
#pragma unroll
  for (int k = 0; k < NV; ++k) {
    const int g = threadIdx.x + k * 256;
    if (g < groups) {
      v[k].x -= mean; v[k].y -= mean; v[k].z -= mean; v[k].w -= mean;
      dev += (v[k].x * v[k].x + v[k].y * v[k].y) + (v[k].z * v[k].z + v[k].w * v[k].w);
    }
  }
  const float scale = 1.f / sqrtf(block_sum(dev, scratch) / (float)width + eps);
  OutT* o = out + (size_t)r * width;
#pragma unroll
  for (int k = 0; k < NV; ++k) {
    const int g = threadIdx.x + k * 256;
    if (g < groups) {
      const float4 w = load4<float>(weight + 4 * g);
      const float4 b = bias ? load4<float>(bias + 4 * g) : make_float4(0.f, 0.f, 0.f, 0.f);
      store4(o + 4 * g, make_float4(v[k].x * scale * w.x + b.x, v[k].y * scale * w.y + b.y, v[k].z * scale * w.z + b.z,
                                    v[k].w * scale * w.w + b.w));
    }
  }
}

template <typename DeltaT, typename OutT>
int launch_add_layernorm(float* x, const void* delta, const float* weight, const float* bias, void* out,
                         const int* rows, int n_rows, int width, float eps, cudaStream_t stream) {
  const bool aligned = width % 4 == 0 && ((uintptr_t)x % 16 == 0) && ((uintptr_t)weight % 16 == 0) &&
                       ((uintptr_t)out % 16 == 0) && (!delta || (uintptr_t)delta % 8 == 0) &&
                       (!bias || (uintptr_t)bias % 16 == 0);
  if (aligned && width <= 4 * 256 * 8) {
    const int groups = width / 4;
    if (groups <= 256 * 2)
      MLL_LAUNCH((add_layernorm_vec_kernel<DeltaT, OutT, 2>), n_rows, 256, 0, stream, x, (const DeltaT*)delta, weight, bias,
                 (OutT*)out, rows, width, eps);
    else if (groups <= 256 * 4)
      MLL_LAUNCH((add_layernorm_vec_kernel<DeltaT, OutT, 4>), n_rows, 256, 0, stream, x, (const DeltaT*)delta, weight, bias,
                 (OutT*)out, rows, width, eps);
    else
      MLL_LAUNCH((add_layernorm_vec_kernel<DeltaT, OutT, 8>), n_rows, 256, 0, stream, x, (const DeltaT*)delta, weight, bias,
                 (OutT*)out, rows, width, eps);
    MLL_LAUNCH_CHECK();
    return 0;
  }
  const int threads = width >= 2048 ? 512 : (width >= 512 ? 256 : 128);
  const size_t smem = (size_t)width * sizeof(float);
  auto kernel = add_layernorm_kernel<DeltaT, OutT>;
  if (smem > 48 * 1024) {
    cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (err != cudaSuccess) {
      mll_set_error("layernorm: cannot reserve %zu bytes of shared memory: %s", smem, cudaGetErrorString(err));
      return (int)err;
    }
  }
  MLL_LAUNCH((kernel), n_rows, threads, smem, stream, x, (const DeltaT*)delta, weight, bias, (OutT*)out, rows, width,
             eps);
  MLL_LAUNCH_CHECK();
  return 0;
}

// Finishes a norm whose rows were left without their factor (RowNormIn), for a product that cannot do
// it itself: out[m, i] = values[m, i] * factor(m).  One block per row.
__global__ void apply_row_norm_kernel(const __nv_bfloat16* __restrict__ values, RowNormIn in,
                                      __nv_bfloat16* __restrict__ out, int width) {
  __shared__ float factor;
  const int m = blockIdx.x;
  if (threadIdx.x < 32) {
    const float f = row_norm_factor<32>(in.sumsq + (size_t)m * in.stride, in.partials, width, in.eps, threadIdx.x,
                                        0xffffffffu);
    if (threadIdx.x == 0) factor = f;
  }
  __syncthreads();
  const float f = factor;
  for (int i = threadIdx.x; i < width; i += blockDim.x)
    out[(size_t)m * width + i] = __float2bfloat16_rn(__bfloat162float(values[(size_t)m * width + i]) * f);
}

}  // namespace mll

// values, out: bfloat16 [n_rows, width]; sumsq: float32 [n_rows, stride] with `partials` sums of squares
// per row; out = values / sqrt(sum / width + eps).
MLL_API int mll_apply_row_norm(const void* values, const float* sumsq, int partials, int stride, float eps, void* out,
                               int n_rows, int width, cudaStream_t stream) {
  MLL_REQUIRE(n_rows >= 0 && width > 0 && partials >= 1 && stride >= partials && eps >= 0.f,
              "apply_row_norm: bad sizes rows=%d width=%d partials=%d stride=%d", n_rows, width, partials, stride);
  if (n_rows == 0) return 0;
  MLL_LAUNCH((mll::apply_row_norm_kernel), n_rows, 256, 0, stream, (const __nv_bfloat16*)values,
             mll::RowNormIn{sumsq, partials, stride, eps}, (__nv_bfloat16*)out, width);
  MLL_LAUNCH_CHECK();
  return 0;
}

MLL_API int mll_add_normed_rmsnorm(float* x, const void* delta, const void* delta2, float scale1, float scale2,
                                   const float* delta_weight, float delta_eps, const float* weight, void* out,
                                   const int* rows, int delta_dtype, int out_dtype, int n_rows, int width, float eps,
                                   cudaStream_t stream);

// x: float32 [*, width] residual stream; delta, delta2: optional [*, width] of `delta_dtype` (delta2 only with
// delta: the outputs of two parts that read the same norm); weight: float32 [width]; out: [n_rows, width] of
// `out_dtype`; rows: optional int32 [n_rows] gather list.  out may be x itself (float32): a block reads its
// whole row before it writes.
MLL_API int mll_add2_rmsnorm(float* x, const void* delta, const void* delta2, const float* weight, void* out,
                             const int* rows, int delta_dtype, int out_dtype, int n_rows, int width, float eps,
                             cudaStream_t stream) {
  return mll_add_normed_rmsnorm(x, delta, delta2, 1.f, 1.f, nullptr, 0.f, weight, out, rows, delta_dtype, out_dtype,
                                n_rows, width, eps, stream);
}

// As mll_add2_rmsnorm with the delta scaled and normalised on its way into the stream:
//   d = scale1 * delta (+ scale2 * delta2);  with delta_weight: d <- d / sqrt(mean(d^2) + delta_eps) * delta_weight;
//   x += d;  out = x / sqrt(mean(x^2) + eps) * weight.   All of it float32.
MLL_API int mll_add_normed_rmsnorm(float* x, const void* delta, const void* delta2, float scale1, float scale2,
                                   const float* delta_weight, float delta_eps, const float* weight, void* out,
                                   const int* rows, int delta_dtype, int out_dtype, int n_rows, int width, float eps,
                                   cudaStream_t stream) {
  MLL_REQUIRE(n_rows >= 0 && width > 0, "rmsnorm: bad sizes rows=%d width=%d", n_rows, width);
  MLL_REQUIRE(delta || !delta_weight, "rmsnorm: a norm of the delta without a delta");
  MLL_REQUIRE(delta_eps >= 0.f, "rmsnorm: the delta's eps must be non-negative");
  const mll::DeltaNorm dn{delta_weight, delta_eps, scale1, scale2};
  MLL_REQUIRE(width <= 50 * 1024, "rmsnorm: width %d exceeds the 51200 floats one block can hold", width);
  MLL_REQUIRE(eps >= 0.f, "rmsnorm: eps must be non-negative");
  MLL_REQUIRE(delta || !delta2, "rmsnorm: a second delta without a first");
  if (n_rows == 0) return 0;
  if (delta_dtype == MLL_F32 && out_dtype == MLL_F32)
    return mll::launch_add_rmsnorm<float, float>(x, delta, delta2, weight, out, rows, n_rows, width, eps, dn, stream);
  if (delta_dtype == MLL_BF16 && out_dtype == MLL_BF16)
    return mll::launch_add_rmsnorm<__nv_bfloat16, __nv_bfloat16>(x, delta, delta2, weight, out, rows, n_rows,
                                                                 width, eps, dn, stream);
  if (delta_dtype == MLL_BF16 && out_dtype == MLL_F32)
    return mll::launch_add_rmsnorm<__nv_bfloat16, float>(x, delta, delta2, weight, out, rows, n_rows, width, eps,
                                                         dn, stream);
  MLL_REQUIRE(false, "rmsnorm: dtypes %d / %d", delta_dtype, out_dtype);
  return -1;
}

MLL_API int mll_add_rmsnorm(float* x, const void* delta, const float* weight, void* out,
                            const int* rows, int act_dtype, int n_rows, int width, float eps,
                            cudaStream_t stream) {
  return mll_add2_rmsnorm(x, delta, nullptr, weight, out, rows, act_dtype, act_dtype, n_rows, width, eps, stream);
}

// Layer norm with weight and (optional) bias after the residual add; arguments as for mll_add2_rmsnorm.
MLL_API int mll_add_layernorm(float* x, const void* delta, const float* weight, const float* bias, void* out,
                              const int* rows, int delta_dtype, int out_dtype, int n_rows, int width, float eps,
                              cudaStream_t stream) {
  MLL_REQUIRE(n_rows >= 0 && width > 0, "layernorm: bad sizes rows=%d width=%d", n_rows, width);
  MLL_REQUIRE(width <= 50 * 1024, "layernorm: width %d exceeds the 51200 floats one block can hold", width);
  MLL_REQUIRE(eps >= 0.f, "layernorm: eps must be non-negative");
  if (n_rows == 0) return 0;
  if (delta_dtype == MLL_F32 && out_dtype == MLL_F32)
    return mll::launch_add_layernorm<float, float>(x, delta, weight, bias, out, rows, n_rows, width, eps, stream);
  if (delta_dtype == MLL_BF16 && out_dtype == MLL_BF16)
    return mll::launch_add_layernorm<__nv_bfloat16, __nv_bfloat16>(x, delta, weight, bias, out, rows, n_rows, width,
                                                                   eps, stream);
  if (delta_dtype == MLL_BF16 && out_dtype == MLL_F32)
    return mll::launch_add_layernorm<__nv_bfloat16, float>(x, delta, weight, bias, out, rows, n_rows, width, eps,
                                                           stream);
  MLL_REQUIRE(false, "layernorm: dtypes %d / %d", delta_dtype, out_dtype);
  return -1;
}
