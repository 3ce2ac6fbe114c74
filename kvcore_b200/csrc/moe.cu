// Mixture of experts: router, grouping of (token, chosen expert) pairs by expert, the experts' two
// matrix products as grouped products over that order, and the weighted sum back per token.
//
//   route:   z = W_router x in 32-bit (one warp per expert row, lane-strided ascending k, butterfly sum);
//            scores = sigmoid(z) or softmax(z); the `top` largest (lowest index among equals); weights are
//            the chosen scores, optionally divided by their sum.  Extra rows (a shared expert's gate) are
//            dotted the same way and leave sigmoid(row . x).
//   align:   pairs p = token * top + slot are laid out expert by expert, each expert's run padded to whole
//            tiles of MOE_BM rows with -1, with the expert of every tile and the number of tiles used.
//            Launch sizes depend on the batch's shape only: blocks beyond the tiles used leave at once.
//   gemm:    out[p, n] = sum_k a(p, k) * w[expert(p), n, k], one accumulator per output taking its
//            products in ascending k, so a pair's result depends on nothing else in the batch.
//            a(p, k) = A[p / a_row_div, k] (* pair weight, rounded to the storage type): the weight
//            multiplies the expert's INPUT.  GATED: w holds gate rows [0, N) and up rows [N, 2N) and
//            out = silu(gate) * up.
//   combine: y[token] = sum over slots of out[token * top + slot] (ascending slot, 32-bit)
//            (+ gate[token] * shared[token]).
#include "common.cuh"

#define MOE_BM 16
#define MOE_BN 64
#define MOE_BK 16
#define MOE_ROUTE_THREADS 128

template <typename T>
__global__ void __launch_bounds__(MOE_ROUTE_THREADS)
moe_route_kernel(int* __restrict__ ids_out, float* __restrict__ weights_out, float* __restrict__ gate_out,
                 const T* __restrict__ x, long long x_stride, const float* __restrict__ router,
                 const float* __restrict__ gate_rows, int E, int R, int K, int top, int score_mode,
                 int renormalize) {
  KVB_KERNEL_PROLOGUE(KVB_TAG_MOE_ROUTE);
  extern __shared__ float smem[];
  float* xs = smem;          // [K]
  float* scores = smem + K;  // [E + R]
  const int token = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = MOE_ROUTE_THREADS / 32;
  const T* row = x + (size_t)token * x_stride;
  for (int k = threadIdx.x; k < K; k += MOE_ROUTE_THREADS) xs[k] = to_float(row[k]);
  __syncthreads();
  for (int e = warp; e < E + R; e += nwarps) {
    const float* w = e < E ? router + (size_t)e * K : gate_rows + (size_t)(e - E) * K;
    float acc = 0.0f;
    for (int k = lane; k < K; k += 32) acc = fmaf(w[k], xs[k], acc);
    acc = warp_sum(acc);
    if (lane == 0) scores[e] = acc;
  }
  __syncthreads();
  if (warp != 0) return;
  for (int r = lane; r < R; r += 32) gate_out[(size_t)token * R + r] = 1.0f / (1.0f + expf(-scores[E + r]));
  if (score_mode == 0) {
    for (int e = lane; e < E; e += 32) scores[e] = 1.0f / (1.0f + expf(-scores[e]));
  } else {
    float m = -INFINITY;
    for (int e = lane; e < E; e += 32) m = fmaxf(m, scores[e]);
    m = warp_max(m);
    float s = 0.0f;
    for (int e = lane; e < E; e += 32) { const float p = expf(scores[e] - m); scores[e] = p; s += p; }
    s = warp_sum(s);
    for (int e = lane; e < E; e += 32) scores[e] = scores[e] / s;
  }
  __syncwarp();
  float chosen_sum = 0.0f;
  for (int slot = 0; slot < top; ++slot) {
    float best = -INFINITY;
    int best_e = 0x7fffffff;
    for (int e = lane; e < E; e += 32) {
      const float v = scores[e];
      if (v > best) { best = v; best_e = e; }   // ascending e: the lowest index among equals stays
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
      if (ov > best || (ov == best && oe < best_e)) { best = ov; best_e = oe; }
    }
    if (lane == 0) {
      ids_out[(size_t)token * top + slot] = best_e;
      weights_out[(size_t)token * top + slot] = best;
      scores[best_e] = -INFINITY;
    }
    chosen_sum += best;
    __syncwarp();
  }
  if (renormalize && lane == 0)
    for (int slot = 0; slot < top; ++slot) weights_out[(size_t)token * top + slot] /= chosen_sum;
}

extern "C" int kvb_moe_route(int* ids_out, float* weights_out, float* gate_out, const void* x, long long x_stride,
                             const float* router, const float* gate_rows, int tokens, int E, int R, int K, int top,
                             int score_mode, int renormalize, int dtype, cudaStream_t stream) {
  if (tokens == 0) return 0;
  KVB_REQUIRE(E > 0 && K > 0 && top > 0 && top <= E, "moe_route: need 0 < top <= experts");
  KVB_REQUIRE(R >= 0 && (R == 0 || (gate_rows != nullptr && gate_out != nullptr)), "moe_route: gate rows need their weights and output");
  KVB_REQUIRE(score_mode == 0 || score_mode == 1, "moe_route: unknown score function");
  const size_t smem = (size_t)(K + E + R) * sizeof(float);
  KVB_REQUIRE(smem <= 200 * 1024, "moe_route: a token's row and scores do not fit in shared memory");
#define KVB_ROUTE(T_)                                                                                          \
  do {                                                                                                         \
    if (smem > 48 * 1024)                                                                                      \
      KVB_CHECK_CUDA(cudaFuncSetAttribute(moe_route_kernel<T_>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
    KVB_CHECK_CUDA(kvb_launch((moe_route_kernel<T_>), dim3(tokens), dim3(MOE_ROUTE_THREADS), smem, stream, true, \
                              ids_out, weights_out, gate_out, (const T_*)x, x_stride, router, gate_rows, E, R, K, \
                              top, score_mode, renormalize));                                                  \
  } while (0)
  if (dtype == KVB_F32) KVB_ROUTE(float); else KVB_ROUTE(bf16);
#undef KVB_ROUTE
  KVB_CHECK_LAUNCH();
  return 0;
}

// sorted [capacity] (capacity = MOE_BM * min(pairs, ceil((pairs + experts * (MOE_BM - 1)) / MOE_BM))),
// tile_expert [capacity / MOE_BM], meta[0] = tiles used.
__global__ void __launch_bounds__(1024)
moe_align_kernel(int* __restrict__ sorted, int* __restrict__ tile_expert, int* __restrict__ meta,
                 const int* __restrict__ ids, int pairs, int E, int capacity, int* status) {
  KVB_KERNEL_PROLOGUE(KVB_TAG_MOE_ALIGN);
  extern __shared__ int ismem[];
  int* counts = ismem;        // [E]
  int* offsets = ismem + E;   // [E]
  for (int e = threadIdx.x; e < E; e += blockDim.x) counts[e] = 0;
  for (int i = threadIdx.x; i < capacity; i += blockDim.x) sorted[i] = -1;
  __syncthreads();
  for (int p = threadIdx.x; p < pairs; p += blockDim.x) {
    const int e = ids[p];
    if (e >= 0 && e < E) atomicAdd(&counts[e], 1);
    else atomicOr(status, KVB_STATUS_BAD_TOKEN);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int at = 0;
    for (int e = 0; e < E; ++e) {
      offsets[e] = at;
      const int tiles = (counts[e] + MOE_BM - 1) / MOE_BM;
      for (int t = 0; t < tiles; ++t) tile_expert[at / MOE_BM + t] = e;
      at += tiles * MOE_BM;
      counts[e] = 0;   // becomes the fill cursor
    }
    meta[0] = at / MOE_BM;
  }
  __syncthreads();
  for (int p = threadIdx.x; p < pairs; p += blockDim.x) {
    const int e = ids[p];
    if (e >= 0 && e < E) sorted[offsets[e] + atomicAdd(&counts[e], 1)] = p;
  }
}

extern "C" int kvb_moe_align(int* sorted, int* tile_expert, int* meta, const int* ids, int pairs, int E,
                             int capacity, cudaStream_t stream) {
  if (pairs == 0) return 0;
  KVB_REQUIRE(E > 0 && E <= 8192, "moe_align: between 1 and 8192 experts");
  // tiles used: one per started run of MOE_BM pairs of an expert, so at most one per pair
  const long long padded = (pairs + (long long)E * (MOE_BM - 1) + MOE_BM - 1) / MOE_BM;
  KVB_REQUIRE(capacity % MOE_BM == 0 && capacity / MOE_BM >= (padded < pairs ? padded : pairs),
              "moe_align: the sorted list is too short");
  int* status = kvb_status_word();
  KVB_REQUIRE(status != nullptr, "moe_align: no status word");
  KVB_CHECK_CUDA(kvb_launch((moe_align_kernel), dim3(1), dim3(1024), (size_t)2 * E * sizeof(int), stream, true,
                            sorted, tile_expert, meta, ids, pairs, E, capacity, status));
  KVB_CHECK_LAUNCH();
  return 0;
}

extern "C" int kvb_moe_tile_rows() { return MOE_BM; }

template <typename T>
__device__ __forceinline__ float moe_silu(float x);
template <>
__device__ __forceinline__ float moe_silu<float>(float x) { return x / (1.0f + expf(-x)); }
template <>
__device__ __forceinline__ float moe_silu<bf16>(float x) { return kvb_silu_for_bf16(x); }

template <typename T, bool GATED>
__global__ void __launch_bounds__(256)
moe_gemm_kernel(T* __restrict__ out, const T* __restrict__ a, long long a_stride, int a_row_div,
                const float* __restrict__ pair_weight, const T* __restrict__ w, const int* __restrict__ sorted,
                const int* __restrict__ tile_expert, const int* __restrict__ meta, int N, int K) {
  KVB_KERNEL_PROLOGUE(KVB_TAG_MOE_GEMM);
  if ((int)blockIdx.x >= meta[0]) return;
  __shared__ float as[MOE_BK][MOE_BM + 1];
  __shared__ float ws[GATED ? 2 : 1][MOE_BK][MOE_BN + 4];
  __shared__ int pair_of[MOE_BM];
  const int expert = tile_expert[blockIdx.x];
  if (threadIdx.x < MOE_BM) pair_of[threadIdx.x] = sorted[blockIdx.x * MOE_BM + threadIdx.x];
  __syncthreads();
  const int n0 = blockIdx.y * MOE_BN;
  const size_t rows_per_expert = (size_t)(GATED ? 2 : 1) * N;
  const T* we = w + (size_t)expert * rows_per_expert * K;
  const int r = threadIdx.x >> 4, c0 = (threadIdx.x & 15) * 4;
  float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f}, acc_up[4] = {0.0f, 0.0f, 0.0f, 0.0f};
  // this thread's element of the A tile: row a_r, column a_k of every slab
  const int a_r = threadIdx.x >> 4, a_k = threadIdx.x & 15;
  const int a_pair = pair_of[a_r];
  const T* a_row = a_pair >= 0 ? a + (size_t)(a_pair / a_row_div) * a_stride : nullptr;
  const float a_scale = (a_pair >= 0 && pair_weight != nullptr) ? pair_weight[a_pair] : 1.0f;
  for (int k0 = 0; k0 < K; k0 += MOE_BK) {
    {
      const int k = k0 + a_k;
      float v = 0.0f;
      if (a_row != nullptr && k < K) {
        v = to_float(a_row[k]);
        if (pair_weight != nullptr) v = to_float(from_float<T>(v * a_scale));
      }
      as[a_k][a_r] = v;
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int idx = threadIdx.x + i * 256;
      const int row = idx >> 4, kk = idx & 15;
      const int n = n0 + row, k = k0 + kk;
      const bool ok = n < N && k < K;
      ws[0][kk][row] = ok ? to_float(we[(size_t)n * K + k]) : 0.0f;
      if (GATED) ws[1][kk][row] = ok ? to_float(we[(size_t)(N + n) * K + k]) : 0.0f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < MOE_BK; ++kk) {
      const float av = as[kk][r];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        acc[j] = fmaf(av, ws[0][kk][c0 + j], acc[j]);
        if (GATED) acc_up[j] = fmaf(av, ws[1][kk][c0 + j], acc_up[j]);
      }
    }
    __syncthreads();
  }
  const int pair = pair_of[r];
  if (pair < 0) return;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int n = n0 + c0 + j;
    if (n >= N) continue;
    float v = acc[j];
    if (GATED) {
      // as the separate kernels would: both products rounded, the activation rounded, then the product
      const float g = to_float(from_float<T>(acc[j])), u = to_float(from_float<T>(acc_up[j]));
      v = to_float(from_float<T>(moe_silu<T>(g))) * u;
    }
    out[(size_t)pair * N + n] = from_float<T>(v);
  }
}

extern "C" int kvb_moe_gemm(void* out, const void* a, long long a_stride, int a_row_div, const float* pair_weight,
                            const void* w, const int* sorted, const int* tile_expert, const int* meta, int max_tiles,
                            int N, int K, int gated, int dtype, cudaStream_t stream) {
  if (max_tiles == 0) return 0;
  KVB_REQUIRE(N > 0 && K > 0 && a_row_div > 0, "moe_gemm: empty product");
  dim3 grid(max_tiles, (N + MOE_BN - 1) / MOE_BN);
  KVB_REQUIRE(grid.y <= 65535, "moe_gemm: too many output columns for one launch");
#define KVB_MOE_GEMM(T_, G_)                                                                                  \
  KVB_CHECK_CUDA(kvb_launch((moe_gemm_kernel<T_, G_>), grid, dim3(256), 0, stream, true, (T_*)out, (const T_*)a, \
                            a_stride, a_row_div, pair_weight, (const T_*)w, sorted, tile_expert, meta, N, K))
  if (dtype == KVB_F32) { if (gated) KVB_MOE_GEMM(float, true); else KVB_MOE_GEMM(float, false); }
  else { if (gated) KVB_MOE_GEMM(bf16, true); else KVB_MOE_GEMM(bf16, false); }
#undef KVB_MOE_GEMM
  KVB_CHECK_LAUNCH();
  return 0;
}

template <typename T>
__global__ void moe_combine_kernel(T* __restrict__ out, const T* __restrict__ expert_out, int top,
                                   const T* __restrict__ shared, const float* __restrict__ gate, int gate_stride,
                                   int width, long long total) {
  KVB_KERNEL_PROLOGUE(KVB_TAG_MOE_COMBINE);
  const long long step = (long long)gridDim.x * blockDim.x;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += step) {
    const long long token = i / width;
    const int col = (int)(i % width);
    float acc = 0.0f;
    for (int slot = 0; slot < top; ++slot) acc += to_float(expert_out[((size_t)token * top + slot) * width + col]);
    if (shared != nullptr) {
      const float s = to_float(shared[i]);
      acc += gate != nullptr ? gate[(size_t)token * gate_stride] * s : s;
    }
    out[i] = from_float<T>(acc);
  }
}

extern "C" int kvb_moe_combine(void* out, const void* expert_out, int tokens, int top, const void* shared,
                               const float* gate, int gate_stride, int width, int dtype, cudaStream_t stream) {
  if (tokens == 0) return 0;
  KVB_REQUIRE(width > 0 && top >= 0, "moe_combine: empty rows");
  const long long total = (long long)tokens * width;
  const int threads = 256;
  const long long wanted = (total + threads - 1) / threads;
  const long long resident = (long long)(kvb_sm_count() > 0 ? kvb_sm_count() : 1) * 16;
  const int blocks = (int)(wanted < resident ? wanted : resident);
  if (dtype == KVB_F32)
    KVB_CHECK_CUDA(kvb_launch((moe_combine_kernel<float>), dim3(blocks), dim3(threads), 0, stream, true, (float*)out,
                              (const float*)expert_out, top, (const float*)shared, gate, gate_stride, width, total));
  else
    KVB_CHECK_CUDA(kvb_launch((moe_combine_kernel<bf16>), dim3(blocks), dim3(threads), 0, stream, true, (bf16*)out,
                              (const bf16*)expert_out, top, (const bf16*)shared, gate, gate_stride, width, total));
  KVB_CHECK_LAUNCH();
  return 0;
}

KVB_TRACE_TU(moe)
