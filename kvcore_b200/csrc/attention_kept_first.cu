// The kept first positions of a sliding-window attention, added to a result that covers the window.
//
// A windowed attention kernel leaves, per (token, head), its normalised output and
//   lse = log2( sum over the window's keys of 2^(score * scale * log2 e) ).
// A query at position p with window w and `keep_first` kept positions also sees the keys
// j < min(keep_first, p - w + 1): those behind its window.  One warp per (token, head) scores them four
// at a time (the lanes spread over the head, 32-bit, online maximum and sum in the same base-2
// domain) and merges:
//   out = (out_w * 2^(lse - M) + sum_j 2^(s_j - M) v_j) / (2^(lse - M) + sum_j 2^(s_j - M)),  M = max(lse, max_j s_j).
// Rows whose window reaches back into the kept positions have nothing to add and are left as they are.
// The kept keys are few (their number is a constant of the model), so this pass costs a small
// fraction of the windowed pass and lets every windowed kernel serve models with kept positions.
#include "common.cuh"

#define AKF_MAX_D 256
#define AKF_WARPS 4

template <typename T>
__global__ void __launch_bounds__(AKF_WARPS * 32)
kept_first_merge_kernel(T* __restrict__ out, int out_stride, const float* __restrict__ lse,
                        const T* __restrict__ q, int q_stride, const T* __restrict__ k_cache,
                        const T* __restrict__ v_cache, const int* __restrict__ table, int table_stride,
                        const int* __restrict__ positions, const int* __restrict__ req_index, int num_rows,
                        int H, int KVH, int D, int page_size, int num_pages, float scale_log2, int window,
                        int keep_first, int* status) {
  KVB_KERNEL_PROLOGUE(KVB_TAG_KEPT_FIRST);
  __shared__ float q_smem[AKF_WARPS][AKF_MAX_D];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row = blockIdx.x * AKF_WARPS + warp;
  if (row >= num_rows) return;
  const int token = row / H, head = row % H;
  const int pos = positions[token];
  const int kept = min(keep_first, pos - window + 1);   // kept keys behind the window
  if (kept <= 0) return;
  const int kvh = head / (H / KVH);
  const int* pages = table + (size_t)req_index[token] * table_stride;
  const T* qrow = q + (size_t)token * q_stride + (size_t)head * D;
  for (int d = lane; d < D; d += 32) q_smem[warp][d] = to_float(qrow[d]);
  __syncwarp();

  constexpr int SLICES = AKF_MAX_D / 32;
  float acc[SLICES];
#pragma unroll
  for (int i = 0; i < SLICES; ++i) acc[i] = 0.0f;
  float running_max = -INFINITY, running_sum = 0.0f;
  const size_t head_off = (size_t)kvh * page_size * D;
  const size_t page_elems = (size_t)KVH * page_size * D;
  // four keys at a time, the lanes spread over the head: every load is a coalesced row of the cache and
  // the four keys' loads and sums are independent of each other
  for (int key0 = 0; key0 < kept; key0 += 4) {
    size_t at[4];
    float dot[4];
    bool live[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int key = key0 + i;
      live[i] = key < kept;
      const int page = live[i] ? pages[key / page_size] : 0;
      if (live[i] && (page <= 0 || page >= num_pages)) {
        if (lane == 0) atomicOr(status, KVB_STATUS_BAD_PAGE);
        live[i] = false;
      }
      at[i] = (size_t)page * page_elems + head_off + (size_t)(key % page_size) * D;
      dot[i] = 0.0f;
    }
    for (int d = lane; d < D; d += 32) {
      const float qd = q_smem[warp][d];
#pragma unroll
      for (int i = 0; i < 4; ++i)
        if (live[i]) dot[i] = fmaf(to_float(k_cache[at[i] + d]), qd, dot[i]);
    }
    float score[4], new_max = running_max;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      score[i] = live[i] ? warp_sum(dot[i]) * scale_log2 : -INFINITY;
      new_max = fmaxf(new_max, score[i]);
    }
    if (new_max == -INFINITY) continue;
    const float correction = (running_max == -INFINITY) ? 0.0f : exp2f(running_max - new_max);
    float p[4];
    running_sum *= correction;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      p[i] = live[i] ? exp2f(score[i] - new_max) : 0.0f;
      running_sum += p[i];
    }
    running_max = new_max;
#pragma unroll
    for (int s = 0; s < SLICES; ++s) {
      const int d = lane + 32 * s;
      if (d < D) {
        float v = acc[s] * correction;
#pragma unroll
        for (int i = 0; i < 4; ++i)
          if (live[i]) v = fmaf(p[i], to_float(v_cache[at[i] + d]), v);
        acc[s] = v;
      }
    }
  }
  if (!(running_sum > 0.0f)) return;
  const float window_lse = lse[(size_t)token * H + head];
  const float top = fmaxf(window_lse, running_max);
  const float w_window = (window_lse == -INFINITY) ? 0.0f : exp2f(window_lse - top);
  const float w_kept = exp2f(running_max - top);
  const float inv = 1.0f / (w_window + running_sum * w_kept);
  T* orow = out + (size_t)token * out_stride + (size_t)head * D;
#pragma unroll
  for (int i = 0; i < SLICES; ++i) {
    const int d = lane + 32 * i;
    if (d < D) orow[d] = from_float<T>((to_float(orow[d]) * w_window + acc[i] * w_kept) * inv);
  }
}

extern "C" int kvb_kept_first_merge(void* out, int out_stride, const float* lse, const void* q, int q_stride,
                                    const void* k_cache, const void* v_cache, const int* table, int table_stride,
                                    const int* positions, const int* req_index, int tokens, int H, int KVH, int D,
                                    int page_size, int num_pages, float scale, int window, int keep_first,
                                    int dtype, cudaStream_t stream) {
  if (tokens == 0 || keep_first <= 0) return 0;
  KVB_REQUIRE(D > 0 && D <= AKF_MAX_D, "kept_first_merge: head_dim must be in [1, 256]");
  KVB_REQUIRE(H > 0 && KVH > 0 && H % KVH == 0, "kept_first_merge: H must be a multiple of KVH");
  KVB_REQUIRE(window > 0 && page_size > 0 && num_pages > 1 && lse != nullptr, "kept_first_merge: needs a window, a cache and the window's sums");
  int* status = kvb_status_word();
  KVB_REQUIRE(status != nullptr, "kept_first_merge: no status word");
  const long long rows = (long long)tokens * H;
  KVB_REQUIRE(rows < (1ll << 31), "kept_first_merge: too many rows");
  const int blocks = (int)((rows + AKF_WARPS - 1) / AKF_WARPS);
  const float scale_log2 = scale * 1.4426950408889634f;
  if (dtype == KVB_F32)
    KVB_CHECK_CUDA(kvb_launch((kept_first_merge_kernel<float>), dim3(blocks), dim3(AKF_WARPS * 32), 0, stream, true,
                              (float*)out, out_stride, lse, (const float*)q, q_stride, (const float*)k_cache,
                              (const float*)v_cache, table, table_stride, positions, req_index, (int)rows, H, KVH, D,
                              page_size, num_pages, scale_log2, window, keep_first, status));
  else
    KVB_CHECK_CUDA(kvb_launch((kept_first_merge_kernel<bf16>), dim3(blocks), dim3(AKF_WARPS * 32), 0, stream, true,
                              (bf16*)out, out_stride, lse, (const bf16*)q, q_stride, (const bf16*)k_cache,
                              (const bf16*)v_cache, table, table_stride, positions, req_index, (int)rows, H, KVH, D,
                              page_size, num_pages, scale_log2, window, keep_first, status));
  KVB_CHECK_LAUNCH();
  return 0;
}

KVB_TRACE_TU(attention_kept_first)
