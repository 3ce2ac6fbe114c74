// Everything between the q/k(/v) projection of a step's tokens and the attention over the paged
// cache, in one kernel: an optional RMS norm of q and of k, a half-layout rotation of the first
// `rot` entries of every head, the write of keys and values into their pages, and q back in place.
//
//   norm_mode 0: none.
//   norm_mode 1: one root mean square over the whole projection (all heads of q at once, all heads of k
//                at once), weights of the projection's size.
//   norm_mode 2: one root mean square per head, weights of the head's size (shared by the heads).
//   value_mode 0: values are the third section of the row (q heads, k heads, v heads).
//   value_mode 1: values are the keys as projected, before the norm and the rotation (row: q heads, k heads).
//
// x * rsqrt(mean(x^2) + eps) * w, sums, angles and rotation are 32-bit; q, the key and the value are
// rounded to the storage type once, at the end.  One block per token; a head's sum of squares is a
// warp's butterfly over a lane-strided walk, and the whole-projection sum adds the heads' sums in
// ascending order, so a token's result does not depend on the batch.
// Cache layout [pages, KVH, page, D]; k_cache == nullptr: nothing is written.
#include "common.cuh"

#define QKP_THREADS 256
// where element i of the token's projections lies in shared memory: four pads after every 32 floats, so that
// threads that each hold 8 neighbouring elements fall into different banks and groups of 4 stay 16-byte aligned
#define QKP_AT(i) ((i) + (((i) >> 5) << 2))

// 8 (or 4) neighbouring 32-bit values of shared memory as 16-byte accesses
template <int N>
__device__ __forceinline__ void qkp_load(float* dst, const float* src) {
#pragma unroll
  for (int q = 0; q < N / 4; ++q) {
    const float4 v = *reinterpret_cast<const float4*>(src + 4 * q);
    dst[4 * q] = v.x; dst[4 * q + 1] = v.y; dst[4 * q + 2] = v.z; dst[4 * q + 3] = v.w;
  }
}
// N norm weights from shared memory (16-byte aligned, N * sizeof(W) a multiple of 16 bytes) as 32-bit values
template <typename W, int N>
__device__ __forceinline__ void qkp_weights(float* dst, const W* src) {
  constexpr int PER = 16 / sizeof(W);
#pragma unroll
  for (int q = 0; q < N / PER; ++q) {
    Vec16<W> v;
    v.load(src + q * PER);
#pragma unroll
    for (int j = 0; j < PER; ++j) dst[q * PER + j] = v.get(j);
  }
}
template <int N>
__device__ __forceinline__ void qkp_store(float* dst, const float* src) {
#pragma unroll
  for (int q = 0; q < N / 4; ++q)
    *reinterpret_cast<float4*>(dst + 4 * q) = make_float4(src[4 * q], src[4 * q + 1], src[4 * q + 2], src[4 * q + 3]);
}

template <typename T, typename W>
__global__ void __launch_bounds__(QKP_THREADS)
qk_prepare_kernel(T* __restrict__ rows, long long row_stride, const int* __restrict__ positions,
                  const int* __restrict__ req_index, const float2* __restrict__ cos_sin,
                  const W* __restrict__ q_weight, const W* __restrict__ k_weight,
                  const int* __restrict__ table, int table_stride, T* __restrict__ k_cache,
                  T* __restrict__ v_cache, int H, int KVH, int D, int rot, int norm_mode, int value_mode,
                  float eps, int page_size, int num_pages, int vec, int* status) {
  KVB_KERNEL_PROLOGUE(KVB_TAG_QK_PREPARE);
  extern __shared__ float smem[];
  const int heads = H + KVH;
  const int half = rot >> 1;
  const bool turn = cos_sin != nullptr && half > 0;
  const int q_len = norm_mode == 1 ? H * D : norm_mode == 2 ? D : 0;
  const int k_len = norm_mode == 1 ? KVH * D : norm_mode == 2 ? D : 0;
  // Everything the later passes need from global memory is asked for before the first barrier: the row,
  // the norm weights, this token's cos/sin and its page; after it the passes run on shared memory alone.
  float* x = smem;                       // [heads * D] (+ one pad after every 32): q heads then k heads, 32-bit
  float* head_sq = smem + QKP_AT((size_t)heads * D) + 4;   // [heads]; what follows starts on a 16-byte boundary
  float2* cs = reinterpret_cast<float2*>(smem + ((QKP_AT((size_t)heads * D) + 4 + heads + 3) & ~(size_t)3));   // [half]
  W* wsm = reinterpret_cast<W*>(cs + ((half + 1) & ~1));    // [q_len + k_len], 16-byte aligned
  // [heads * D / VN] sums of squares, one per vector of the load pass (vector path with a norm only)
  float* part = reinterpret_cast<float*>(reinterpret_cast<unsigned char*>(wsm) + (((size_t)(q_len + k_len) * sizeof(W) + 15) & ~(size_t)15));
  const int token = blockIdx.x;
  const int pos = positions[token];
  T* row = rows + (size_t)token * row_stride;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = QKP_THREADS / 32;
  constexpr int VN = Vec16<T>::N;   // `vec`: rows, heads and cache rows start on 16-byte boundaries
  // the last pass takes whole vectors (and their rotation partners) when the turned half is made of whole vectors
  const bool fused = vec && (!turn || half % VN == 0) && (VN * sizeof(W)) % 16 == 0;

  size_t cache_base = 0;
  bool write = k_cache != nullptr;
  if (write) {
    const int page = table[(size_t)req_index[token] * table_stride + pos / page_size];
    if (page <= 0 || page >= num_pages) {
      if (threadIdx.x == 0) atomicOr(status, KVB_STATUS_BAD_PAGE);
      write = false;
    }
    cache_base = ((size_t)page * KVH * page_size + (pos % page_size)) * D;
  }
  const size_t head_stride = (size_t)page_size * D;
  if (vec) {
    for (int i = threadIdx.x * VN; i < heads * D; i += QKP_THREADS * VN) {
      Vec16<T> v;
      v.load(row + i);
      float f[VN], sq = 0.0f;
#pragma unroll
      for (int j = 0; j < VN; ++j) { f[j] = v.get(j); sq = fmaf(f[j], f[j], sq); }
      qkp_store<VN>(x + QKP_AT(i), f);
      if (norm_mode != 0) part[i / VN] = sq;
    }
  } else {
    for (int i = threadIdx.x; i < heads * D; i += QKP_THREADS) x[QKP_AT(i)] = to_float(row[i]);
  }
  constexpr int WN = Vec16<W>::N;
  if (fused && q_len % WN == 0 && k_len % WN == 0 && aligned16(q_weight) && aligned16(k_weight)) {
    for (int i = threadIdx.x * WN; i < q_len + k_len; i += QKP_THREADS * WN) {
      Vec16<W> w;
      w.load(i < q_len ? q_weight + i : k_weight + (i - q_len));
      w.store(wsm + i);
    }
  } else {
    for (int i = threadIdx.x; i < q_len + k_len; i += QKP_THREADS) wsm[i] = i < q_len ? q_weight[i] : k_weight[i - q_len];
  }
  if (turn)
    for (int j = threadIdx.x; j < half; j += QKP_THREADS) cs[j] = cos_sin[(size_t)token * half + j];
  if (write && value_mode == 0) {      // values of their own: a copy that depends on nothing else here
    const T* v = row + (size_t)(H + KVH) * D;
    if (vec) {
      for (int i = threadIdx.x * VN; i < KVH * D; i += QKP_THREADS * VN) {
        Vec16<T> t;
        t.load(v + i);
        t.store(v_cache + cache_base + (size_t)(i / D) * head_stride + i % D);
      }
    } else {
      for (int i = threadIdx.x; i < KVH * D; i += QKP_THREADS)
        v_cache[cache_base + (size_t)(i / D) * head_stride + i % D] = v[i];
    }
  }
  __syncthreads();

  if (write && value_mode == 1) {      // the values are the keys as projected: exact in 32-bit, stored back as they were
    const int step = vec ? VN : 1;
    for (int i = threadIdx.x * step; i < KVH * D; i += QKP_THREADS * step) {
      T* dst = v_cache + cache_base + (size_t)(i / D) * head_stride + i % D;
      if (vec) {
        Vec16<T> t;
#pragma unroll
        for (int j = 0; j < VN; ++j) t.set(j, x[QKP_AT(H * D + i + j)]);
        t.store(dst);
      } else {
        dst[0] = from_float<T>(x[QKP_AT(H * D + i)]);
      }
    }
  }

  if (norm_mode != 0) {
    for (int h = warp; h < heads; h += nwarps) {
      float sq = 0.0f;
      if (vec) {     // the vectors' sums of the load pass, lane-strided over the head's vectors
        const int per_head = D / VN;
        for (int v = lane; v < per_head; v += 32) sq += part[h * per_head + v];
      } else {
        for (int d = lane; d < D; d += 32) { const float v = x[QKP_AT(h * D + d)]; sq = fmaf(v, v, sq); }
      }
      sq = warp_sum(sq);
      if (lane == 0) head_sq[h] = sq;
    }
    __syncthreads();
    float q_inv = 0.0f, k_inv = 0.0f;
    if (norm_mode == 1) {
      // every warp adds the heads' sums the same way: lane l takes heads l, l + 32, ... in ascending order,
      // then the butterfly
      float q_sq = 0.0f, k_sq = 0.0f;
      for (int h = lane; h < H; h += 32) q_sq += head_sq[h];
      for (int h = H + lane; h < heads; h += 32) k_sq += head_sq[h];
      q_sq = warp_sum(q_sq);
      k_sq = warp_sum(k_sq);
      q_inv = 1.0f / sqrtf(q_sq / (float)(H * D) + eps);
      k_inv = KVH > 0 ? 1.0f / sqrtf(k_sq / (float)(KVH * D) + eps) : 0.0f;
    }
    if (fused) {
      // The vector pass below scales on the fly: value(i) = x[i] * scale(head) * w(i).
      // A vector and its rotation partner lie in one head; `base + j` addresses element i + j (a vector of 8
      // never crosses a pad).
      for (int i = threadIdx.x * VN; i < heads * D; i += QKP_THREADS * VN) {
        const int h = i / D, d = i - h * D;
        const float scale = norm_mode == 1 ? (h < H ? q_inv : k_inv) : 1.0f / sqrtf(head_sq[h] / (float)D + eps);
        const int w_at = norm_mode == 1 ? i : (h < H ? d : q_len + d);
        float own[VN], wv[VN];
        qkp_load<VN>(own, x + QKP_AT(i));
        qkp_weights<W, VN>(wv, wsm + w_at);
#pragma unroll
        for (int j = 0; j < VN; ++j) own[j] *= scale * wv[j];
        Vec16<T> v;
        if (turn && d < rot) {
          const bool low = d < half;
          const int mate = low ? half : -half;
          float other[VN], t[2 * VN];
          qkp_load<VN>(other, x + QKP_AT(i + mate));
          qkp_weights<W, VN>(wv, wsm + w_at + mate);
          qkp_load<2 * VN>(t, reinterpret_cast<const float*>(cs + (low ? d : d - half)));   // (cos, sin) pairs
#pragma unroll
          for (int j = 0; j < VN; ++j) {
            const float o = other[j] * scale * wv[j];
            v.set(j, low ? own[j] * t[2 * j] - o * t[2 * j + 1] : own[j] * t[2 * j] + o * t[2 * j + 1]);
          }
        } else {
#pragma unroll
          for (int j = 0; j < VN; ++j) v.set(j, own[j]);
        }
        v.store(row + i);
        if (h >= H && write) v.store(k_cache + cache_base + (size_t)(h - H) * head_stride + d);
      }
      return;
    }
    for (int i = threadIdx.x; i < heads * D; i += QKP_THREADS) {
      const int h = i / D, d = i % D;
      const float scale = norm_mode == 1 ? (h < H ? q_inv : k_inv) : 1.0f / sqrtf(head_sq[h] / (float)D + eps);
      const int at = norm_mode == 1 ? i : (h < H ? d : q_len + d);
      x[QKP_AT(i)] = x[QKP_AT(i)] * scale * to_float(wsm[at]);
    }
  }
  __syncthreads();   // (also: the values were copied from what is overwritten from here on)

  if (fused) {
    // no norm: rotation and store in one pass, a vector of the turned part taking its partner from shared memory
    for (int i = threadIdx.x * VN; i < heads * D; i += QKP_THREADS * VN) {
      const int h = i / D, d = i - h * D;
      const int base = QKP_AT(i);
      Vec16<T> v;
      if (turn && d < rot) {
        const bool low = d < half;
        const int mate_base = QKP_AT(low ? i + half : i - half);
        const float2* t = cs + (low ? d : d - half);
#pragma unroll
        for (int j = 0; j < VN; ++j)
          v.set(j, low ? x[base + j] * t[j].x - x[mate_base + j] * t[j].y : x[base + j] * t[j].x + x[mate_base + j] * t[j].y);
      } else {
#pragma unroll
        for (int j = 0; j < VN; ++j) v.set(j, x[base + j]);
      }
      v.store(row + i);
      if (h >= H && write) v.store(k_cache + cache_base + (size_t)(h - H) * head_stride + d);
    }
    return;
  }
  if (turn) {
    for (int item = threadIdx.x; item < heads * half; item += QKP_THREADS) {
      const int h = item / half, j = item % half;
      const float2 t = cs[j];
      const int lo = h * D + j, hi = lo + half;
      const float a = x[QKP_AT(lo)], b = x[QKP_AT(hi)];
      x[QKP_AT(lo)] = a * t.x - b * t.y;
      x[QKP_AT(hi)] = b * t.x + a * t.y;
    }
    __syncthreads();
  }
  for (int i = threadIdx.x; i < heads * D; i += QKP_THREADS) {
    const T v = from_float<T>(x[QKP_AT(i)]);
    row[i] = v;
    if (i >= H * D && write) {
      const int kh = (i - H * D) / D, d = (i - H * D) % D;
      k_cache[cache_base + (size_t)kh * head_stride + d] = v;
    }
  }
}

// The same work for rows that are made of whole 16-byte vectors and few enough of them that a thread can keep
// its own (at most QKP_REG_VECTORS) in registers from the load to the store: the row, the norm weights of a
// thread's vectors and of their rotation partners are asked for at once; shared memory only carries the raw row
// (for the partners of the rotation and the values), the vectors' sums of squares and this token's cos/sin.
#define QKP_REG_VECTORS 3
template <typename T, typename W>
__global__ void __launch_bounds__(QKP_THREADS, 4)
qk_prepare_regs_kernel(T* __restrict__ rows, long long row_stride, const int* __restrict__ positions,
                       const int* __restrict__ req_index, const float2* __restrict__ cos_sin,
                       const W* __restrict__ q_weight, const W* __restrict__ k_weight,
                       const int* __restrict__ table, int table_stride, T* __restrict__ k_cache,
                       T* __restrict__ v_cache, int H, int KVH, int D, int rot, int norm_mode, int value_mode,
                       float eps, int page_size, int num_pages, int* status) {
  KVB_KERNEL_PROLOGUE(KVB_TAG_QK_PREPARE);
  extern __shared__ __align__(16) unsigned char regs_smem[];
  constexpr int VN = Vec16<T>::N;
  const int heads = H + KVH, total = heads * D, nvec = total / VN;
  const int half = rot >> 1;
  const bool turn = cos_sin != nullptr && half > 0;
  const int q_len = norm_mode == 1 ? H * D : D;
  T* raw = reinterpret_cast<T*>(regs_smem);                                   // [total]
  float* part = reinterpret_cast<float*>(raw + total);                        // [nvec]
  float* head_sq = part + ((nvec + 3) & ~3);                                  // [max(heads, 2 * warps)]
  float2* cs = reinterpret_cast<float2*>(head_sq + ((max(heads, 2 * (QKP_THREADS / 32)) + 3) & ~3));   // [half]
  const int token = blockIdx.x;
  const int pos = positions[token];
  T* row = rows + (size_t)token * row_stride;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = QKP_THREADS / 32;

  size_t cache_base = 0;
  bool write = k_cache != nullptr;
  if (write) {
    const int page = table[(size_t)req_index[token] * table_stride + pos / page_size];
    if (page <= 0 || page >= num_pages) {
      if (threadIdx.x == 0) atomicOr(status, KVB_STATUS_BAD_PAGE);
      write = false;
    }
    cache_base = ((size_t)page * KVH * page_size + (pos % page_size)) * D;
  }
  const size_t head_stride = (size_t)page_size * D;

  Vec16<T> mine[QKP_REG_VECTORS];
  Vec16<W> w_own[QKP_REG_VECTORS], w_mate[QKP_REG_VECTORS];
#pragma unroll
  for (int n = 0; n < QKP_REG_VECTORS; ++n) {
    const int i = (threadIdx.x + n * QKP_THREADS) * VN;
    if (i < total) {
      mine[n].load(row + i);
      if (norm_mode != 0) {
        const int h = i / D, d = i - h * D;
        const int at = norm_mode == 1 ? i : (h < H ? d : q_len + d);
        w_own[n].load(at < q_len ? q_weight + at : k_weight + (at - q_len));
        if (turn && d < rot) {
          const int mate = at + (d < half ? half : -half);
          w_mate[n].load(mate < q_len ? q_weight + mate : k_weight + (mate - q_len));
        }
      }
    }
  }
  if (turn)
    for (int j = threadIdx.x; j < half; j += QKP_THREADS) cs[j] = cos_sin[(size_t)token * half + j];
  if (write && value_mode == 0) {
    const T* v = row + (size_t)(H + KVH) * D;
    for (int i = threadIdx.x * VN; i < KVH * D; i += QKP_THREADS * VN) {
      Vec16<T> t;
      t.load(v + i);
      t.store(v_cache + cache_base + (size_t)(i / D) * head_stride + i % D);
    }
  }
  float my_q = 0.0f, my_k = 0.0f;      // this thread's share of the two sums of squares (its vectors in order)
#pragma unroll
  for (int n = 0; n < QKP_REG_VECTORS; ++n) {
    const int i = (threadIdx.x + n * QKP_THREADS) * VN;
    if (i < total) {
      mine[n].store(raw + i);
      float sq = 0.0f;
#pragma unroll
      for (int j = 0; j < VN; ++j) { const float f = mine[n].get(j); sq = fmaf(f, f, sq); }
      if (norm_mode == 2) part[i / VN] = sq;
      if (i < H * D) my_q += sq; else my_k += sq;
    }
  }
  if (norm_mode == 1) {                // one barrier: a butterfly per warp, then the warps' sums in ascending order
    my_q = warp_sum(my_q);
    my_k = warp_sum(my_k);
    if (lane == 0) { head_sq[warp] = my_q; head_sq[nwarps + warp] = my_k; }
  }
  __syncthreads();

  if (write && value_mode == 1) {      // the values are the keys as projected
    for (int i = threadIdx.x * VN; i < KVH * D; i += QKP_THREADS * VN) {
      Vec16<T> t;
      t.load(raw + H * D + i);
      t.store(v_cache + cache_base + (size_t)(i / D) * head_stride + i % D);
    }
  }
  float q_inv = 1.0f, k_inv = 1.0f;
  if (norm_mode == 1) {
    float q_sq = 0.0f, k_sq = 0.0f;
#pragma unroll
    for (int wi = 0; wi < QKP_THREADS / 32; ++wi) { q_sq += head_sq[wi]; k_sq += head_sq[QKP_THREADS / 32 + wi]; }
    q_inv = 1.0f / sqrtf(q_sq / (float)(H * D) + eps);
    k_inv = KVH > 0 ? 1.0f / sqrtf(k_sq / (float)(KVH * D) + eps) : 0.0f;
  } else if (norm_mode == 2) {
    const int per_head = D / VN;
    for (int h = warp; h < heads; h += nwarps) {
      float sq = 0.0f;
      for (int v = lane; v < per_head; v += 32) sq += part[h * per_head + v];
      sq = warp_sum(sq);
      if (lane == 0) head_sq[h] = sq;
    }
    __syncthreads();
  }
#pragma unroll
  for (int n = 0; n < QKP_REG_VECTORS; ++n) {
    const int i = (threadIdx.x + n * QKP_THREADS) * VN;
    if (i >= total) continue;
    const int h = i / D, d = i - h * D;
    float scale = 1.0f;
    if (norm_mode == 1) scale = h < H ? q_inv : k_inv;
    else if (norm_mode == 2) scale = 1.0f / sqrtf(head_sq[h] / (float)D + eps);
    float own[VN];
#pragma unroll
    for (int j = 0; j < VN; ++j) own[j] = norm_mode != 0 ? mine[n].get(j) * scale * w_own[n].get(j) : mine[n].get(j);
    Vec16<T> v;
    if (turn && d < rot) {
      const bool low = d < half;
      Vec16<T> m;
      m.load(raw + i + (low ? half : -half));
      float t[2 * VN];
      qkp_load<2 * VN>(t, reinterpret_cast<const float*>(cs + (low ? d : d - half)));
#pragma unroll
      for (int j = 0; j < VN; ++j) {
        const float o = norm_mode != 0 ? m.get(j) * scale * w_mate[n].get(j) : m.get(j);
        v.set(j, low ? own[j] * t[2 * j] - o * t[2 * j + 1] : own[j] * t[2 * j] + o * t[2 * j + 1]);
      }
    } else {
#pragma unroll
      for (int j = 0; j < VN; ++j) v.set(j, own[j]);
    }
    v.store(row + i);
    if (h >= H && write) v.store(k_cache + cache_base + (size_t)(h - H) * head_stride + d);
  }
}

extern "C" int kvb_qk_prepare(void* rows, long long row_stride, const int* positions, const int* req_index,
                              const float* cos_sin, const void* q_weight, const void* k_weight, const int* table,
                              int table_stride, void* k_cache, void* v_cache, int tokens, int H, int KVH, int D,
                              int rot, int norm_mode, int value_mode, float eps, int page_size, int num_pages,
                              int dtype, int weight_dtype, cudaStream_t stream) {
  if (tokens == 0) return 0;
  KVB_REQUIRE(D > 0 && H >= 0 && KVH >= 0 && H + KVH > 0, "qk_prepare: no heads");
  KVB_REQUIRE(rot >= 0 && rot <= D && rot % 2 == 0, "qk_prepare: the rotated entries must be an even count within the head");
  KVB_REQUIRE(norm_mode >= 0 && norm_mode <= 2, "qk_prepare: unknown norm mode");
  KVB_REQUIRE(value_mode == 0 || value_mode == 1, "qk_prepare: unknown value mode");
  KVB_REQUIRE(norm_mode == 0 || (q_weight != nullptr && (KVH == 0 || k_weight != nullptr)), "qk_prepare: a norm needs its weights");
  KVB_REQUIRE((k_cache == nullptr) == (v_cache == nullptr), "qk_prepare: give both caches or none");
  KVB_REQUIRE(k_cache == nullptr || (table != nullptr && page_size > 0 && KVH > 0), "qk_prepare: a cache write needs a block table");
  const long long needed = (long long)(H + KVH + (k_cache != nullptr && value_mode == 0 ? KVH : 0)) * D;
  KVB_REQUIRE(row_stride >= needed, "qk_prepare: row stride is smaller than the row");
  int* status = kvb_status_word();
  KVB_REQUIRE(status != nullptr, "qk_prepare: no status word");
  const size_t elems = (size_t)(H + KVH) * D;
  const size_t norm_len = norm_mode == 1 ? elems : norm_mode == 2 ? 2 * (size_t)D : 0;
  const size_t smem = (QKP_AT(elems) + 8 + (size_t)(H + KVH)) * sizeof(float) + (size_t)(rot / 2 + 2) * sizeof(float2) +
                      norm_len * (weight_dtype == KVB_F32 ? 4 : 2) + 16 + (norm_mode != 0 ? elems / 4 + 1 : 0) * sizeof(float);
  KVB_REQUIRE(smem <= 200 * 1024, "qk_prepare: the projections of one token do not fit in shared memory");
  const int esize = dtype == KVB_F32 ? 4 : 2;
  const int vec = ((size_t)D * esize) % 16 == 0 && ((size_t)row_stride * esize) % 16 == 0 && aligned16(rows) &&
                  (k_cache == nullptr || (aligned16(k_cache) && aligned16(v_cache)));
  const int vn = 16 / esize;
  const bool weights_ok = norm_mode == 0 || (dtype == weight_dtype && aligned16(q_weight) && (KVH == 0 || aligned16(k_weight)));
  const bool in_registers = vec && weights_ok && (rot == 0 || cos_sin == nullptr || (rot / 2) % vn == 0) &&
                            elems <= (size_t)QKP_THREADS * QKP_REG_VECTORS * vn;
  const size_t nvec = elems / vn;
  const size_t regs_smem = elems * esize + (((nvec + 3) & ~(size_t)3) + (((size_t)(H + KVH) + 2 * (QKP_THREADS / 32) + 3) & ~(size_t)3)) * sizeof(float) +
                           (size_t)(rot / 2 + 2) * sizeof(float2);
#define KVB_QKP_REGS(T_, W_)                                                                                \
  do {                                                                                                      \
    if (regs_smem > 48 * 1024)                                                                              \
      KVB_CHECK_CUDA(cudaFuncSetAttribute(qk_prepare_regs_kernel<T_, W_>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)regs_smem)); \
    KVB_CHECK_CUDA(kvb_launch((qk_prepare_regs_kernel<T_, W_>), dim3(tokens), dim3(QKP_THREADS), regs_smem, stream, true, \
                              (T_*)rows, row_stride, positions, req_index, (const float2*)cos_sin,          \
                              (const W_*)q_weight, (const W_*)k_weight, table, table_stride, (T_*)k_cache,  \
                              (T_*)v_cache, H, KVH, D, rot, norm_mode, value_mode, eps, page_size, num_pages, status)); \
  } while (0)
  if (in_registers) {
    if (dtype == KVB_F32) KVB_QKP_REGS(float, float); else KVB_QKP_REGS(bf16, bf16);
    KVB_CHECK_LAUNCH();
    return 0;
  }
#undef KVB_QKP_REGS
#define KVB_QKP(T_, W_)                                                                                     \
  do {                                                                                                      \
    if (smem > 48 * 1024)                                                                                   \
      KVB_CHECK_CUDA(cudaFuncSetAttribute(qk_prepare_kernel<T_, W_>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
    KVB_CHECK_CUDA(kvb_launch((qk_prepare_kernel<T_, W_>), dim3(tokens), dim3(QKP_THREADS), smem, stream, true, \
                              (T_*)rows, row_stride, positions, req_index, (const float2*)cos_sin,          \
                              (const W_*)q_weight, (const W_*)k_weight, table, table_stride, (T_*)k_cache,  \
                              (T_*)v_cache, H, KVH, D, rot, norm_mode, value_mode, eps, page_size, num_pages, vec, status)); \
  } while (0)
  if (dtype == KVB_F32) {
    KVB_REQUIRE(weight_dtype == KVB_F32, "qk_prepare: a 32-bit model needs 32-bit norm weights");
    KVB_QKP(float, float);
  } else if (weight_dtype == KVB_F32) {
    KVB_QKP(bf16, float);
  } else {
    KVB_QKP(bf16, bf16);
  }
#undef KVB_QKP
  KVB_CHECK_LAUNCH();
  return 0;
}

KVB_TRACE_TU(qk_prepare)
