// Layer norm over a 32-bit (or 16-bit) residual stream, and the sum that keeps that stream.
//
//   layer_norm: y = (x - mean) / sqrt(var + eps) * w (+ b), var = mean((x - mean)^2); the mean, the
//   deviations, the variance and the scaling are 32-bit whatever the storage types.  One block of
//   256 threads per row: the reduction tree depends on the width only, so a row's result does not
//   depend on the rest of the batch.  Input, output and weight types are independent (a 32-bit
//   stream normalised into bf16 activations is the serving case).
//
//   stream_add: out = base + (a + b) in 32-bit, base and out 32-bit (in place allowed), a and b of
//   the activation type; with base of the activation type and no a, b it widens rows into a stream.
#include "common.cuh"

#define LN_THREADS 256
#define LN_KEEP 16   // values a thread keeps in registers between the passes (rows up to 4,096 wide)

// Rows whose width is a multiple of 4 and at most 4,096, on 16-byte boundaries: a thread holds 4 neighbouring
// columns per pass (one 16-byte load of a 32-bit row), the same three passes over registers.
template <typename IN, typename OUT, typename W>
__global__ void __launch_bounds__(LN_THREADS)
layer_norm_vec4_kernel(OUT* __restrict__ out, const IN* __restrict__ x, const W* __restrict__ weight,
                       const W* __restrict__ bias, int width, float eps) {
  KVB_KERNEL_PROLOGUE(KVB_TAG_LAYERNORM);
  __shared__ float scratch[32];
  const IN* row = x + (size_t)blockIdx.x * width;
  OUT* orow = out + (size_t)blockIdx.x * width;
  constexpr int PASSES = LN_KEEP / 4;
  float mine[PASSES][4];
  float sum = 0.0f;
#pragma unroll
  for (int s = 0; s < PASSES; ++s) {
    const int i = (threadIdx.x + s * LN_THREADS) * 4;
    if (i < width) {
      if (sizeof(IN) == 4) {
        const float4 v = *reinterpret_cast<const float4*>(row + i);
        mine[s][0] = v.x; mine[s][1] = v.y; mine[s][2] = v.z; mine[s][3] = v.w;
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j) mine[s][j] = to_float(row[i + j]);
      }
    } else {
      mine[s][0] = mine[s][1] = mine[s][2] = mine[s][3] = 0.0f;
    }
    sum += (mine[s][0] + mine[s][1]) + (mine[s][2] + mine[s][3]);
  }
  const float mean = block_sum(sum, scratch) / (float)width;
  float sq = 0.0f;
#pragma unroll
  for (int s = 0; s < PASSES; ++s) {
    const int i = (threadIdx.x + s * LN_THREADS) * 4;
    if (i < width) {
#pragma unroll
      for (int j = 0; j < 4; ++j) { const float d = mine[s][j] - mean; sq = fmaf(d, d, sq); }
    }
  }
  const float var = block_sum(sq, scratch) / (float)width;
  const float inv = 1.0f / sqrtf(var + eps);
#pragma unroll
  for (int s = 0; s < PASSES; ++s) {
    const int i = (threadIdx.x + s * LN_THREADS) * 4;
    if (i < width) {
      float y[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        y[j] = (mine[s][j] - mean) * inv * to_float(weight[i + j]);
        if (bias != nullptr) y[j] += to_float(bias[i + j]);
      }
      if (sizeof(OUT) == 4) {
        *reinterpret_cast<float4*>(orow + i) = make_float4(y[0], y[1], y[2], y[3]);
      } else {
        __nv_bfloat162 lo = __floats2bfloat162_rn(y[0], y[1]), hi = __floats2bfloat162_rn(y[2], y[3]);
        uint2 packed;
        packed.x = *reinterpret_cast<unsigned*>(&lo);
        packed.y = *reinterpret_cast<unsigned*>(&hi);
        *reinterpret_cast<uint2*>(orow + i) = packed;
      }
    }
  }
}

template <typename IN, typename OUT, typename W>
__global__ void __launch_bounds__(LN_THREADS)
layer_norm_kernel(OUT* __restrict__ out, const IN* __restrict__ x, const W* __restrict__ weight,
                  const W* __restrict__ bias, int width, float eps) {
  KVB_KERNEL_PROLOGUE(KVB_TAG_LAYERNORM);
  __shared__ float scratch[32];
  const IN* row = x + (size_t)blockIdx.x * width;
  OUT* orow = out + (size_t)blockIdx.x * width;
  const bool kept = width <= LN_THREADS * LN_KEEP;
  float mine[LN_KEEP];
  float sum = 0.0f;
  if (kept) {
#pragma unroll
    for (int s = 0; s < LN_KEEP; ++s) {
      const int i = threadIdx.x + s * LN_THREADS;
      mine[s] = i < width ? to_float(row[i]) : 0.0f;
      sum += mine[s];
    }
  } else {
    for (int i = threadIdx.x; i < width; i += LN_THREADS) sum += to_float(row[i]);
  }
  const float mean = block_sum(sum, scratch) / (float)width;
  float sq = 0.0f;
  if (kept) {
#pragma unroll
    for (int s = 0; s < LN_KEEP; ++s) {
      const int i = threadIdx.x + s * LN_THREADS;
      const float d = i < width ? mine[s] - mean : 0.0f;
      sq += d * d;
    }
  } else {
    for (int i = threadIdx.x; i < width; i += LN_THREADS) {
      const float d = to_float(row[i]) - mean;
      sq += d * d;
    }
  }
  const float var = block_sum(sq, scratch) / (float)width;
  const float inv = 1.0f / sqrtf(var + eps);
  if (kept) {
#pragma unroll
    for (int s = 0; s < LN_KEEP; ++s) {
      const int i = threadIdx.x + s * LN_THREADS;
      if (i < width) {
        float y = (mine[s] - mean) * inv * to_float(weight[i]);
        if (bias != nullptr) y += to_float(bias[i]);
        orow[i] = from_float<OUT>(y);
      }
    }
  } else {
    for (int i = threadIdx.x; i < width; i += LN_THREADS) {
      float y = (to_float(row[i]) - mean) * inv * to_float(weight[i]);
      if (bias != nullptr) y += to_float(bias[i]);
      orow[i] = from_float<OUT>(y);
    }
  }
}

template <typename IN, typename OUT, typename W>
static cudaError_t launch_layer_norm(void* out, const void* x, const void* w, const void* b, int rows, int width,
                                     float eps, cudaStream_t stream) {
  if (width % 4 == 0 && width <= LN_THREADS * LN_KEEP && aligned16(out) && aligned16(x))
    return kvb_launch((layer_norm_vec4_kernel<IN, OUT, W>), dim3(rows), dim3(LN_THREADS), 0, stream, true,
                      (OUT*)out, (const IN*)x, (const W*)w, (const W*)b, width, eps);
  return kvb_launch((layer_norm_kernel<IN, OUT, W>), dim3(rows), dim3(LN_THREADS), 0, stream, true,
                    (OUT*)out, (const IN*)x, (const W*)w, (const W*)b, width, eps);
}

extern "C" int kvb_layer_norm(void* out, const void* x, const void* weight, const void* bias, int rows, int width,
                              float eps, int in_dtype, int out_dtype, int weight_dtype, cudaStream_t stream) {
  if (rows == 0) return 0;
  KVB_REQUIRE(width > 0, "layer_norm: width must be positive");
  const int code = (in_dtype == KVB_BF16 ? 4 : 0) | (out_dtype == KVB_BF16 ? 2 : 0) | (weight_dtype == KVB_BF16 ? 1 : 0);
  cudaError_t err;
  switch (code) {
    case 0: err = launch_layer_norm<float, float, float>(out, x, weight, bias, rows, width, eps, stream); break;
    case 1: err = launch_layer_norm<float, float, bf16>(out, x, weight, bias, rows, width, eps, stream); break;
    case 2: err = launch_layer_norm<float, bf16, float>(out, x, weight, bias, rows, width, eps, stream); break;
    case 3: err = launch_layer_norm<float, bf16, bf16>(out, x, weight, bias, rows, width, eps, stream); break;
    case 4: err = launch_layer_norm<bf16, float, float>(out, x, weight, bias, rows, width, eps, stream); break;
    case 5: err = launch_layer_norm<bf16, float, bf16>(out, x, weight, bias, rows, width, eps, stream); break;
    case 6: err = launch_layer_norm<bf16, bf16, float>(out, x, weight, bias, rows, width, eps, stream); break;
    default: err = launch_layer_norm<bf16, bf16, bf16>(out, x, weight, bias, rows, width, eps, stream); break;
  }
  KVB_CHECK_CUDA(err);
  KVB_CHECK_LAUNCH();
  return 0;
}

template <typename BASE, typename T>
__global__ void stream_add_kernel(float* __restrict__ out, const BASE* __restrict__ base, const T* __restrict__ a,
                                  const T* __restrict__ b, long long count) {
  KVB_KERNEL_PROLOGUE(KVB_TAG_STREAM_ADD);
  const long long step = (long long)gridDim.x * blockDim.x;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < count; i += step) {
    float v = to_float(base[i]);
    if (a != nullptr) {
      float s = to_float(a[i]);
      if (b != nullptr) s += to_float(b[i]);
      v += s;
    }
    out[i] = v;
  }
}

// out (32-bit) = base + (a + b); base is 32-bit (base_dtype KVB_F32) or of the activation type.
extern "C" int kvb_stream_add(float* out, const void* base, int base_dtype, const void* a, const void* b,
                              long long count, int dtype, cudaStream_t stream) {
  if (count == 0) return 0;
  KVB_REQUIRE(out != nullptr && base != nullptr, "stream_add: no stream");
  KVB_REQUIRE(a != nullptr || b == nullptr, "stream_add: a second addend needs a first");
  const int threads = 256;
  const long long wanted = (count + threads - 1) / threads;
  const long long resident = (long long)(kvb_sm_count() > 0 ? kvb_sm_count() : 1) * 16;
  const int blocks = (int)(wanted < resident ? wanted : resident);
  cudaError_t err;
  if (base_dtype == KVB_F32 && dtype == KVB_F32)
    err = kvb_launch((stream_add_kernel<float, float>), dim3(blocks), dim3(threads), 0, stream, true, out,
                     (const float*)base, (const float*)a, (const float*)b, count);
  else if (base_dtype == KVB_F32)
    err = kvb_launch((stream_add_kernel<float, bf16>), dim3(blocks), dim3(threads), 0, stream, true, out,
                     (const float*)base, (const bf16*)a, (const bf16*)b, count);
  else
    err = kvb_launch((stream_add_kernel<bf16, bf16>), dim3(blocks), dim3(threads), 0, stream, true, out,
                     (const bf16*)base, (const bf16*)a, (const bf16*)b, count);
  KVB_CHECK_CUDA(err);
  KVB_CHECK_LAUNCH();
  return 0;
}

KVB_TRACE_TU(layer_norm)
