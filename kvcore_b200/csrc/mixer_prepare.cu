// Small kernels between the projections and the attention of two mixers, 32-bit inside, one rounding at
// the store.
//
//   latent_prepare (latent attention: one cached vector a token).  A projected row holds `rank` latent
//   entries and `rot` position entries.  The latent entries get an RMS norm with a weight; the position
//   entries are turned by the token's position, entry 2i with entry 2i+1 (interleaved pairs), angle
//   position * inv_freq[i], for the first `dims` of them.  Both go into the token's cached row
//   [rank | rot].  The query rows [heads, width + rot] get the same turn on their last `rot` entries,
//   written behind the `rank` entries of the attention's query rows [heads, rank + rot]; the first
//   `rank` entries of those rows (the query carried into the latent space) are copied from `q_latent`
//   when given, else left as the caller filled them.
//
//   head_norm_kv_write (attention with several score maps a head).  q and k are cut into vectors of
//   `dim` entries (one per head and map); each gets an RMS norm of its own with one weight shared by
//   all; q is normed in place, the normed k and the values go side by side into the token's cached row
//   [k | v].
//
//   maps_combine: o = a1 - lambda * a2 of the two maps of a head (32-bit in), divided by its root mean
//   square over the head's values, times a constant; written in the activation type.
//
//   sigmoid_gate_mul: out[t, h, :] = o[t, h, :] * sigmoid(g[t, h, :]), o with strides of its own.
#include "common.cuh"

#define MP_THREADS 128
#define LP_HEADS 8      // query heads a block of latent_prepare handles

template <typename T>
__global__ void __launch_bounds__(MP_THREADS)
latent_prepare_kernel(const T* __restrict__ kv_rows, long long kv_stride, const T* __restrict__ norm_weight,
                      float eps, const float* __restrict__ inv_freq, int dims, const int* __restrict__ positions,
                      const int* __restrict__ req_index, const int* __restrict__ table, int table_stride,
                      T* __restrict__ cache, int page_size, int num_pages, int write, const T* __restrict__ q,
                      long long q_token_stride, long long q_head_stride, int q_width,
                      const T* __restrict__ q_latent, long long ql_token_stride, long long ql_head_stride,
                      T* __restrict__ q_out, int heads, int rank, int rot, int lead, int* status) {
  KVB_KERNEL_PROLOGUE(KVB_TAG_LATENT_PREPARE);
  __shared__ float scratch[32];
  const int t = blockIdx.x;
  const int pos = positions[t];
  const float fpos = (float)pos;
  const int row_width = rank + rot;     // of a cached row
  const int q_row = lead + rot;         // of a row of q_out: `lead` entries the caller fills or q_latent gives, then the turned part
  // blockIdx.y: a group of LP_HEADS query heads, or (the last one) the token's cached row
  if (blockIdx.y == gridDim.y - 1) {
    if (!write) return;
    const T* src = kv_rows + (size_t)t * kv_stride;
    float ss = 0.0f;
    for (int i = threadIdx.x; i < rank; i += MP_THREADS) {
      const float v = to_float(src[i]);
      ss = fmaf(v, v, ss);
    }
    const float inv = 1.0f / sqrtf(block_sum(ss, scratch) / (float)rank + eps);
    const int page = table[(size_t)req_index[t] * table_stride + pos / page_size];
    if (page <= 0 || page >= num_pages) {
      if (threadIdx.x == 0) atomicOr(status, KVB_STATUS_BAD_PAGE);
    } else {
      T* dst = cache + ((size_t)page * page_size + pos % page_size) * row_width;
      for (int i = threadIdx.x; i < rank; i += MP_THREADS)
        dst[i] = from_float<T>(to_float(src[i]) * inv * to_float(norm_weight[i]));
      for (int i = threadIdx.x; i < rot / 2; i += MP_THREADS) {
        float u = to_float(src[rank + 2 * i]), v = to_float(src[rank + 2 * i + 1]);
        if (2 * i < dims) {
          float s, c;
          sincosf(fpos * inv_freq[i], &s, &c);
          const float nu = u * c - v * s, nv = v * c + u * s;
          u = nu; v = nv;
        }
        dst[rank + 2 * i] = from_float<T>(u);
        dst[rank + 2 * i + 1] = from_float<T>(v);
      }
      if ((rot & 1) && threadIdx.x == 0) dst[rank + rot - 1] = src[rank + rot - 1];
    }
    return;
  }
  // query rows of LP_HEADS heads: the turned position part behind the leading part.  The angles depend on
  // the token only: their cos/sin are made once a block.
  __shared__ float cs[2][MP_THREADS];
  const int h0 = blockIdx.y * LP_HEADS, h1 = min(heads, h0 + LP_HEADS);
  const int pairs = rot / 2;
  for (int base = 0; base < pairs; base += MP_THREADS) {
    const int mine = base + threadIdx.x;
    if (mine < pairs) {
      float s = 0.0f, c = 1.0f;
      if (2 * mine < dims) sincosf(fpos * inv_freq[mine], &s, &c);
      cs[0][threadIdx.x] = c;
      cs[1][threadIdx.x] = s;
    }
    __syncthreads();
    const int here = min(MP_THREADS, pairs - base);
    for (int i = threadIdx.x; i < (h1 - h0) * here; i += MP_THREADS) {
      const int h = h0 + i / here, j = i % here;
      const T* src = q + (size_t)t * q_token_stride + (size_t)h * q_head_stride + q_width + 2 * (base + j);
      const float u = to_float(src[0]), v = to_float(src[1]);
      T* dst = q_out + ((size_t)t * heads + h) * q_row + lead + 2 * (base + j);
      dst[0] = from_float<T>(u * cs[0][j] - v * cs[1][j]);
      dst[1] = from_float<T>(v * cs[0][j] + u * cs[1][j]);
    }
    __syncthreads();
  }
  if (rot & 1)
    for (int h = h0 + threadIdx.x; h < h1; h += MP_THREADS)
      q_out[((size_t)t * heads + h) * q_row + lead + rot - 1] =
          q[(size_t)t * q_token_stride + (size_t)h * q_head_stride + q_width + rot - 1];
  if (q_latent != nullptr) {
    constexpr int N = Vec16<T>::N;
    const bool vec = lead % N == 0 && q_row % N == 0 && ql_token_stride % N == 0 && ql_head_stride % N == 0 &&
                     aligned16(q_latent) && aligned16(q_out);
    const int per = vec ? lead / N : lead;
    for (int i = threadIdx.x; i < (h1 - h0) * per; i += MP_THREADS) {
      const int h = h0 + i / per, j = (i % per) * (vec ? N : 1);
      const T* src = q_latent + (size_t)t * ql_token_stride + (size_t)h * ql_head_stride + j;
      T* dst = q_out + ((size_t)t * heads + h) * q_row + j;
      if (vec) {
        Vec16<T> v;
        v.load(src);
        v.store(dst);
      } else {
        *dst = *src;
      }
    }
  }
}

extern "C" int kvb_latent_prepare(const void* kv_rows, long long kv_stride, const void* norm_weight, float eps,
                                  const float* inv_freq, int dims, const int* positions, const int* req_index,
                                  const int* table, int table_stride, void* cache, int page_size, int num_pages,
                                  int write, const void* q, long long q_token_stride, long long q_head_stride,
                                  int q_width, const void* q_latent, long long ql_token_stride,
                                  long long ql_head_stride, void* q_out, int tokens, int heads, int rank, int rot,
                                  int lead, int dtype, cudaStream_t stream) {
  if (tokens == 0) return 0;
  KVB_REQUIRE(rank > 0 && rot >= 0 && heads > 0 && heads < 65535 && dims >= 0 && dims <= rot && dims % 2 == 0 &&
              lead > 0, "latent_prepare: bad sizes");
  int* status = kvb_status_word();
  KVB_REQUIRE(status != nullptr, "latent_prepare: no status word");
  if (dtype == KVB_F32)
    KVB_CHECK_CUDA(kvb_launch((latent_prepare_kernel<float>), dim3(tokens, (heads + LP_HEADS - 1) / LP_HEADS + 1), dim3(MP_THREADS), 0, stream, true,
        (const float*)kv_rows, kv_stride, (const float*)norm_weight, eps, inv_freq, dims, positions, req_index, table,
        table_stride, (float*)cache, page_size, num_pages, write, (const float*)q, q_token_stride, q_head_stride,
        q_width, (const float*)q_latent, ql_token_stride, ql_head_stride, (float*)q_out, heads, rank, rot, lead, status));
  else
    KVB_CHECK_CUDA(kvb_launch((latent_prepare_kernel<bf16>), dim3(tokens, (heads + LP_HEADS - 1) / LP_HEADS + 1), dim3(MP_THREADS), 0, stream, true,
        (const bf16*)kv_rows, kv_stride, (const bf16*)norm_weight, eps, inv_freq, dims, positions, req_index, table,
        table_stride, (bf16*)cache, page_size, num_pages, write, (const bf16*)q, q_token_stride, q_head_stride,
        q_width, (const bf16*)q_latent, ql_token_stride, ql_head_stride, (bf16*)q_out, heads, rank, rot, lead, status));
  KVB_CHECK_LAUNCH();
  return 0;
}

// Rows of a cache that keeps one row a token, brought together: entry n of the lists names a request (row of
// the block table) and a position; columns [col0, col0 + cols) of that token's cached row go to
// dst[n * dst_row_stride + h * dst_head_stride + 0..cols) for every h < copies.
template <typename T>
__global__ void __launch_bounds__(MP_THREADS)
gather_cached_rows_kernel(T* __restrict__ dst, long long dst_row_stride, long long dst_head_stride, int copies,
                          const T* __restrict__ cache, int row_width, int col0, int cols,
                          const int* __restrict__ src_req, const int* __restrict__ src_pos,
                          const int* __restrict__ table, int table_stride, int page_size, int num_pages, int* status) {
  KVB_KERNEL_PROLOGUE(KVB_TAG_GATHER_CACHED);
  const int n = blockIdx.x;
  const int pos = src_pos[n];
  const int page = table[(size_t)src_req[n] * table_stride + pos / page_size];
  if (page <= 0 || page >= num_pages) {
    if (threadIdx.x == 0) atomicOr(status, KVB_STATUS_BAD_PAGE);
    return;
  }
  const T* src = cache + ((size_t)page * page_size + pos % page_size) * row_width + col0;
  T* out = dst + (size_t)n * dst_row_stride;
  constexpr int N = Vec16<T>::N;
  const bool vec = cols % N == 0 && col0 % N == 0 && row_width % N == 0 && dst_row_stride % N == 0 &&
                   dst_head_stride % N == 0 && aligned16(cache) && aligned16(dst);
  if (vec) {
    const int chunks = cols / N;
    for (int i = threadIdx.x; i < copies * chunks; i += MP_THREADS) {
      const int h = i / chunks, c = (i % chunks) * N;
      Vec16<T> v;
      v.load(src + c);
      v.store(out + (size_t)h * dst_head_stride + c);
    }
  } else {
    for (int i = threadIdx.x; i < copies * cols; i += MP_THREADS) {
      const int h = i / cols, c = i % cols;
      out[(size_t)h * dst_head_stride + c] = src[c];
    }
  }
}

extern "C" int kvb_gather_cached_rows(void* dst, long long dst_row_stride, long long dst_head_stride, int copies,
                                      const void* cache, int row_width, int col0, int cols, const int* src_req,
                                      const int* src_pos, int count, const int* table, int table_stride,
                                      int page_size, int num_pages, int dtype, cudaStream_t stream) {
  if (count == 0) return 0;
  KVB_REQUIRE(copies > 0 && cols > 0 && col0 >= 0 && col0 + cols <= row_width, "gather_cached_rows: bad columns");
  int* status = kvb_status_word();
  KVB_REQUIRE(status != nullptr, "gather_cached_rows: no status word");
  if (dtype == KVB_F32)
    KVB_CHECK_CUDA(kvb_launch((gather_cached_rows_kernel<float>), dim3(count), dim3(MP_THREADS), 0, stream, true,
        (float*)dst, dst_row_stride, dst_head_stride, copies, (const float*)cache, row_width, col0, cols, src_req,
        src_pos, table, table_stride, page_size, num_pages, status));
  else
    KVB_CHECK_CUDA(kvb_launch((gather_cached_rows_kernel<bf16>), dim3(count), dim3(MP_THREADS), 0, stream, true,
        (bf16*)dst, dst_row_stride, dst_head_stride, copies, (const bf16*)cache, row_width, col0, cols, src_req,
        src_pos, table, table_stride, page_size, num_pages, status));
  KVB_CHECK_LAUNCH();
  return 0;
}

// Four neighbouring entries, loaded and stored as one access.
template <typename T>
struct __align__(4 * sizeof(T)) Quad { T v[4]; };
#define HN_KEEP 4     // quads a lane keeps of a vector (vectors up to 512 entries; longer ones go entry by entry)

template <typename T>
__global__ void __launch_bounds__(MP_THREADS)
head_norm_kv_write_kernel(T* __restrict__ rows, long long row_stride, const T* __restrict__ q_weight,
                          const T* __restrict__ k_weight, float eps, const int* __restrict__ positions,
                          const int* __restrict__ req_index, const int* __restrict__ table, int table_stride,
                          T* __restrict__ cache, int page_size, int num_pages, int write, int q_vectors,
                          int k_vectors, int dim, int v_width, int per_block, int* status) {
  KVB_KERNEL_PROLOGUE(KVB_TAG_HEAD_NORM_KV);
  const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  T* row = rows + (size_t)t * row_stride;
  T* dst = nullptr;
  if (write) {
    const int pos = positions[t];
    const int page = table[(size_t)req_index[t] * table_stride + pos / page_size];
    if (page <= 0 || page >= num_pages) {
      if (threadIdx.x == 0 && blockIdx.y == 0) atomicOr(status, KVB_STATUS_BAD_PAGE);
    } else {
      dst = cache + ((size_t)page * page_size + pos % page_size) * ((size_t)k_vectors * dim + v_width);
    }
  }
  const int vectors = q_vectors + (write ? k_vectors : 0);
  // four neighbouring entries a lane and load where the vectors allow it (8 bytes of bf16, 16 of float)
  const bool quads = dim % 4 == 0 && v_width % 4 == 0 && row_stride % 4 == 0 &&
                     (reinterpret_cast<uintptr_t>(rows) % (4 * sizeof(T))) == 0 &&
                     (reinterpret_cast<uintptr_t>(cache) % (4 * sizeof(T))) == 0 &&
                     (reinterpret_cast<uintptr_t>(q_weight) % (4 * sizeof(T))) == 0 &&
                     (k_weight == nullptr || (reinterpret_cast<uintptr_t>(k_weight) % (4 * sizeof(T))) == 0);
  // blockIdx.y: a group of `per_block` vectors (one a warp at a time); the block of the first group also copies
  // the values
  const int group_end = min(vectors, (int)(blockIdx.y + 1) * per_block);
  for (int n = blockIdx.y * per_block + warp; n < group_end; n += MP_THREADS / 32) {
    const bool is_q = n < q_vectors;
    T* vec = row + (size_t)n * dim;
    const T* w = is_q ? q_weight : k_weight;
    T* o = is_q ? vec : (dst == nullptr ? nullptr : dst + (size_t)(n - q_vectors) * dim);
    float ss = 0.0f;
    if (quads && dim <= 4 * 32 * HN_KEEP) {
      Quad<T> mine[HN_KEEP];
#pragma unroll
      for (int s = 0; s < HN_KEEP; ++s) {
        const int i = (lane + 32 * s) * 4;
        if (i < dim) {
          mine[s] = *reinterpret_cast<const Quad<T>*>(vec + i);
#pragma unroll
          for (int j = 0; j < 4; ++j) { const float v = to_float(mine[s].v[j]); ss = fmaf(v, v, ss); }
        }
      }
      const float inv = 1.0f / sqrtf(warp_sum(ss) / (float)dim + eps);
      if (o != nullptr) {
#pragma unroll
        for (int s = 0; s < HN_KEEP; ++s) {
          const int i = (lane + 32 * s) * 4;
          if (i < dim) {
            const Quad<T> wq = *reinterpret_cast<const Quad<T>*>(w + i);
            Quad<T> r;
#pragma unroll
            for (int j = 0; j < 4; ++j) r.v[j] = from_float<T>(to_float(mine[s].v[j]) * inv * to_float(wq.v[j]));
            *reinterpret_cast<Quad<T>*>(o + i) = r;
          }
        }
      }
      continue;
    }
    for (int i = lane; i < dim; i += 32) {
      const float v = to_float(vec[i]);
      ss = fmaf(v, v, ss);
    }
    const float inv = 1.0f / sqrtf(warp_sum(ss) / (float)dim + eps);
    if (o != nullptr)
      for (int i = lane; i < dim; i += 32) o[i] = from_float<T>(to_float(vec[i]) * inv * to_float(w[i]));
  }
  if (dst != nullptr && blockIdx.y == 0) {
    const T* v = row + (size_t)(q_vectors + k_vectors) * dim;
    T* out = dst + (size_t)k_vectors * dim;
    if (quads) {
      for (int i = threadIdx.x * 4; i < v_width; i += MP_THREADS * 4)
        *reinterpret_cast<Quad<T>*>(out + i) = *reinterpret_cast<const Quad<T>*>(v + i);
    } else {
      for (int i = threadIdx.x; i < v_width; i += MP_THREADS) out[i] = v[i];
    }
  }
}

extern "C" int kvb_head_norm_kv_write(void* rows, long long row_stride, const void* q_weight, const void* k_weight,
                                      float eps, const int* positions, const int* req_index, const int* table,
                                      int table_stride, void* cache, int page_size, int num_pages, int write,
                                      int tokens, int q_vectors, int k_vectors, int dim, int v_width, int dtype,
                                      cudaStream_t stream) {
  if (tokens == 0) return 0;
  KVB_REQUIRE(q_vectors > 0 && k_vectors > 0 && dim > 0 && v_width > 0, "head_norm_kv_write: bad sizes");
  int* status = kvb_status_word();
  KVB_REQUIRE(status != nullptr, "head_norm_kv_write: no status word");
  // few tokens (decoding): four vectors a block, so that the step's few rows spread over the GPU; many tokens: a
  // block a token walks all its vectors (a block of one vector a warp is over before it has paid for its launch)
  const int vectors = q_vectors + (write ? k_vectors : 0);
  const int per_block = tokens >= 512 ? ((vectors + 3) / 4) * 4 : MP_THREADS / 32;
  const int groups = (vectors + per_block - 1) / per_block;
  KVB_REQUIRE(groups <= 65535, "head_norm_kv_write: too many vectors a token");
  if (dtype == KVB_F32)
    KVB_CHECK_CUDA(kvb_launch((head_norm_kv_write_kernel<float>), dim3(tokens, groups), dim3(MP_THREADS), 0, stream, true,
        (float*)rows, row_stride, (const float*)q_weight, (const float*)k_weight, eps, positions, req_index, table,
        table_stride, (float*)cache, page_size, num_pages, write, q_vectors, k_vectors, dim, v_width, per_block, status));
  else
    KVB_CHECK_CUDA(kvb_launch((head_norm_kv_write_kernel<bf16>), dim3(tokens, groups), dim3(MP_THREADS), 0, stream, true,
        (bf16*)rows, row_stride, (const bf16*)q_weight, (const bf16*)k_weight, eps, positions, req_index, table,
        table_stride, (bf16*)cache, page_size, num_pages, write, q_vectors, k_vectors, dim, v_width, per_block, status));
  KVB_CHECK_LAUNCH();
  return 0;
}

template <typename T>
__global__ void __launch_bounds__(MP_THREADS)
maps_combine_kernel(T* __restrict__ out, const float* __restrict__ a, long long rows, int width, float lambda,
                    float eps, float out_scale) {
  KVB_KERNEL_PROLOGUE(KVB_TAG_MAPS_COMBINE);
  const long long row = (long long)blockIdx.x * (MP_THREADS / 32) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  const float* a1 = a + (size_t)row * 2 * width;
  const float* a2 = a1 + width;
  float ss = 0.0f;
  for (int i = lane; i < width; i += 32) {
    const float o = a1[i] - lambda * a2[i];
    ss = fmaf(o, o, ss);
  }
  const float mul = out_scale / sqrtf(warp_sum(ss) / (float)width + eps);
  for (int i = lane; i < width; i += 32) out[(size_t)row * width + i] = from_float<T>((a1[i] - lambda * a2[i]) * mul);
}

extern "C" int kvb_maps_combine(void* out, const float* a, long long rows, int width, float lambda, float eps,
                                float out_scale, int dtype, cudaStream_t stream) {
  if (rows == 0) return 0;
  KVB_REQUIRE(width > 0, "maps_combine: width must be positive");
  const long long blocks = (rows + MP_THREADS / 32 - 1) / (MP_THREADS / 32);
  KVB_REQUIRE(blocks < (1ll << 31), "maps_combine: too many rows");
  if (dtype == KVB_F32)
    KVB_CHECK_CUDA(kvb_launch((maps_combine_kernel<float>), dim3((unsigned)blocks), dim3(MP_THREADS), 0, stream, true,
                              (float*)out, a, rows, width, lambda, eps, out_scale));
  else
    KVB_CHECK_CUDA(kvb_launch((maps_combine_kernel<bf16>), dim3((unsigned)blocks), dim3(MP_THREADS), 0, stream, true,
                              (bf16*)out, a, rows, width, lambda, eps, out_scale));
  KVB_CHECK_LAUNCH();
  return 0;
}

template <typename T, bool VEC>
__global__ void sigmoid_gate_mul_kernel(T* __restrict__ out, const T* __restrict__ o, long long o_token_stride,
                                        long long o_head_stride, const T* __restrict__ g, long long g_stride,
                                        long long count, int heads, int width) {
  KVB_KERNEL_PROLOGUE(KVB_TAG_GATE_MUL);
  constexpr int N = VEC ? Vec16<T>::N : 1;     // entries a thread handles at once (they never straddle a head)
  const long long step = (long long)gridDim.x * blockDim.x;
  const int per_token = heads * width;
  for (long long i = (blockIdx.x * (long long)blockDim.x + threadIdx.x) * N; i < count; i += step * N) {
    const long long t = i / per_token;
    const int c = (int)(i % per_token), h = c / width, j = c % width;
    const T* value = o + t * o_token_stride + (long long)h * o_head_stride + j;
    const T* gate = g + t * g_stride + c;
    if (VEC) {
      Vec16<T> a, b;
      a.load(value);
      b.load(gate);
#pragma unroll
      for (int n = 0; n < N; ++n) a.set(n, a.get(n) / (1.0f + __expf(-b.get(n))));
      a.store(out + i);
    } else {
      out[i] = from_float<T>(to_float(*value) / (1.0f + expf(-to_float(*gate))));
    }
  }
}

extern "C" int kvb_sigmoid_gate_mul(void* out, const void* o, long long o_token_stride, long long o_head_stride,
                                    const void* g, long long g_stride, int tokens, int heads, int width, int dtype,
                                    cudaStream_t stream) {
  const long long count = (long long)tokens * heads * width;
  if (count == 0) return 0;
  const int threads = 256;
  const long long wanted = (count / (dtype == KVB_BF16 ? 8 : 1) + threads - 1) / threads + 1;
  const long long resident = (long long)(kvb_sm_count() > 0 ? kvb_sm_count() : 1) * 16;
  const int blocks = (int)(wanted < resident ? wanted : resident);
  // bf16 rows made of 16-byte vectors: eight entries a thread (the activation type's rounding hides the fast
  // exponential); everything else one entry a thread with the exact one
  const bool vec = dtype == KVB_BF16 && width % 8 == 0 && o_token_stride % 8 == 0 && o_head_stride % 8 == 0 &&
                   g_stride % 8 == 0 && aligned16(out) && aligned16(o) && aligned16(g);
  if (dtype == KVB_F32)
    KVB_CHECK_CUDA(kvb_launch((sigmoid_gate_mul_kernel<float, false>), dim3(blocks), dim3(threads), 0, stream, true,
        (float*)out, (const float*)o, o_token_stride, o_head_stride, (const float*)g, g_stride, count, heads, width));
  else if (vec)
    KVB_CHECK_CUDA(kvb_launch((sigmoid_gate_mul_kernel<bf16, true>), dim3(blocks), dim3(threads), 0, stream, true,
        (bf16*)out, (const bf16*)o, o_token_stride, o_head_stride, (const bf16*)g, g_stride, count, heads, width));
  else
    KVB_CHECK_CUDA(kvb_launch((sigmoid_gate_mul_kernel<bf16, false>), dim3(blocks), dim3(threads), 0, stream, true,
        (bf16*)out, (const bf16*)o, o_token_stride, o_head_stride, (const bf16*)g, g_stride, count, heads, width));
  KVB_CHECK_LAUNCH();
  return 0;
}

KVB_TRACE_TU(mixer_prepare)
