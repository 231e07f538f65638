// Several residual streams side by side (hyper-connections), and what surrounds them:
//
//  * embedding gather (+ a learned vector per position) into `streams` float32 copies of the
//    residual stream, laid out [token][stream][hidden];
//  * the kernel every sublayer boundary of such a model is: apply the previous sublayer's
//    not-yet-applied write to all streams (new_t = sum_s mix[s][t] old_s + out[t] * y), read the
//    next sublayer's input (u = sum_t read[t] new_t), and RMS-normalise it with a gain vector or a
//    single gain.  With one stream and no weights this is residual add + RMSNorm.
//  * q/k normalised over their whole projection, value heads divided by their root mean square,
//    and the write of keys and values into the paged cache.
//
// All sums, statistics and the streams themselves are float32; a result is rounded once to the
// activation type.  A row's result depends on that row alone.
#include "common.cuh"

CIE_DEFINE_LAST_ERROR()

namespace cie {

constexpr int kMaxStreams = 16;

// ---------------------------------------------------------------- embedding
template <typename T>
__global__ void embedding_streams_kernel(const int* __restrict__ ids, const int* __restrict__ positions,
                                         const T* __restrict__ table, const T* __restrict__ position_table,
                                         float* __restrict__ residual, int hidden, int vocab,
                                         int max_positions, int streams, float scale, int* err) {
  pdl_wait();
  pdl_trigger();
  const int t = blockIdx.x;
  int id = ids[t];
  if (id < 0 || id >= vocab) {
    if (threadIdx.x == 0) atomicOr(err, kErrBadToken);
    id = 0;
  }
  const T* row = table + (size_t)id * hidden;
  const T* prow = nullptr;
  if (position_table) {
    int p = positions[t];
    if (p < 0 || p >= max_positions) {
      if (threadIdx.x == 0) atomicOr(err, kErrBadToken);
      p = 0;
    }
    prow = position_table + (size_t)p * hidden;
  }
  float* out = residual + (size_t)t * streams * hidden;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    float v = to_float(row[i]) * scale;
    if (prow) v += to_float(prow[i]);
    for (int s = 0; s < streams; ++s) out[(size_t)s * hidden + i] = v;
  }
}

// ---------------------------------------------------------------- streams: write, read, normalise
// One block per output row.  rows == nullptr: row r is token r and the streams are updated in
// place.  rows != nullptr: row r reads token rows[r]; nothing is written back.
//   update   y [tokens][hidden] (TU: float or the activation type), or nullptr (nothing pending)
//   mix      [S][S] indexed [from][to], or nullptr (identity)
//   out_w    [S], or nullptr (ones)
//   read     [S], or nullptr (ones: the plain sum of the streams)
//   gain     [hidden], or one number when gain_single
// MAXS: the most streams the instance takes (its loops are unrolled to that many).
template <typename T, typename TU, int MAXS>
__global__ void __launch_bounds__(256) stream_norm_kernel(float* __restrict__ streams, int S, const TU* __restrict__ update,
                                   const float* __restrict__ mix, const float* __restrict__ out_w,
                                   const float* __restrict__ read, const float* __restrict__ gain,
                                   int gain_single, T* __restrict__ out, const int* __restrict__ rows,
                                   int hidden, float eps) {
  extern __shared__ float u_s[];          // the row that is normalised
  __shared__ float scratch[33];
  __shared__ float mix_s[kMaxStreams * kMaxStreams], out_s[kMaxStreams], read_s[kMaxStreams];
  pdl_trigger();   // what follows is a matrix product that only asks for weights before its own wait
  pdl_wait();
  for (int e = threadIdx.x; e < S * S; e += blockDim.x) mix_s[e] = mix ? mix[e] : (e / S == e % S ? 1.f : 0.f);
  if (threadIdx.x < S) {
    out_s[threadIdx.x] = out_w ? out_w[threadIdx.x] : 1.f;
    read_s[threadIdx.x] = read ? read[threadIdx.x] : 1.f;
  }
  __syncthreads();
  const int r = blockIdx.x;
  const int src = rows ? rows[r] : r;
  float* base = streams + (size_t)src * S * hidden;
  const TU* y_row = update ? update + (size_t)src * hidden : nullptr;
  const bool write_back = rows == nullptr && update != nullptr;
  float sumsq = 0.f;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    float x[MAXS];
#pragma unroll
    for (int s = 0; s < MAXS; ++s) x[s] = s < S ? base[(size_t)s * hidden + i] : 0.f;
    float u = 0.f;
    if (y_row) {
      const float y = to_float(y_row[i]);
#pragma unroll
      for (int t = 0; t < MAXS; ++t) {
        if (t >= S) break;
        float v = 0.f;
#pragma unroll
        for (int s = 0; s < MAXS; ++s)
          if (s < S) v = fmaf(mix_s[s * S + t], x[s], v);
        v = fmaf(out_s[t], y, v);
        if (write_back) base[(size_t)t * hidden + i] = v;
        u = fmaf(read_s[t], v, u);
      }
    } else {
#pragma unroll
      for (int t = 0; t < MAXS; ++t)
        if (t < S) u = fmaf(read_s[t], x[t], u);
    }
    u_s[i] = u;
    sumsq = fmaf(u, u, sumsq);
  }
  const float total = block_sum(sumsq, scratch);
  const float inv = rsqrtf(total / (float)hidden + eps);
  T* dst = out + (size_t)r * hidden;
  const float single = gain_single ? gain[0] : 0.f;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x)
    dst[i] = from_float<T>((gain_single ? single : gain[i]) * (u_s[i] * inv));
}

// ---------------------------------------------------------------- q/k/v: norms, rotation and cache write
// One block per token.  The source row is [q_heads*dim | kv_heads*dim | kv_heads*vdim] (+ bias), of the
// activation type or float32 (a product's float32 result that is not rounded before the norm).
//   qk_norm  1: q and k are each divided by the root mean square of their WHOLE projection (all heads
//            together) and multiplied by a gain vector of that size; 2: every head by its own root mean
//            square, times a gain vector of a head's size that all heads share
//   v_norm   every value head is divided by its own root mean square (no gain)
//   rotation (inv_freq != nullptr) after the norms the first rot_dims elements of every q and k head turn by
//            position * inv_freq[i], pair (i, i + rot_dims / 2) or, interleaved, (2i, 2i + 1); cos and sin
//            are multiplied by `magnitude`; angle and rotation float32
// q goes to q_out (row stride q_stride); k and v go to their page slots
// ([page][kv_head][page_size][dim or vdim]).
template <typename TI, typename T>
__global__ void norm_kv_write_kernel(const TI* __restrict__ src, const float* __restrict__ bias,
                                     T* __restrict__ q_out, int q_stride,
                                     const int* __restrict__ positions,
                                     const int* __restrict__ request_of_token,
                                     const int* __restrict__ table, int table_width, int num_pages,
                                     T* __restrict__ k_pool, T* __restrict__ v_pool,
                                     const float* __restrict__ q_gain, const float* __restrict__ k_gain,
                                     int q_heads, int kv_heads, int dim, int vdim, int page_size,
                                     int qk_norm, int v_norm, float eps, int write_cache, int src_stride,
                                     const float* __restrict__ inv_freq, int rot_dims, float magnitude,
                                     int interleaved, int* err) {
  extern __shared__ float row_s[];
  __shared__ float scratch[33];
  pdl_wait();
  pdl_trigger();
  const int t = blockIdx.x;
  const int q_width = q_heads * dim, k_width = kv_heads * dim, v_width = kv_heads * vdim;
  const int width = q_width + k_width + v_width;
  const TI* row = src + (size_t)t * src_stride;
  float sq_q = 0.f, sq_k = 0.f;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    float v = to_float(row[i]);
    if (bias) v += bias[i];
    row_s[i] = v;
    if (i < q_width) sq_q = fmaf(v, v, sq_q);
    else if (i < q_width + k_width) sq_k = fmaf(v, v, sq_k);
  }
  __syncthreads();
  if (qk_norm == 1) {
    const float inv_q = rsqrtf(block_sum(sq_q, scratch) / (float)q_width + eps);
    const float inv_k = rsqrtf(block_sum(sq_k, scratch) / (float)k_width + eps);
    for (int i = threadIdx.x; i < q_width + k_width; i += blockDim.x)
      row_s[i] = i < q_width ? q_gain[i] * (row_s[i] * inv_q) : k_gain[i - q_width] * (row_s[i] * inv_k);
    __syncthreads();
  } else if (qk_norm == 2) {
    // every q and k head by its own root mean square, times a gain vector of the head's size that all heads
    // share; a warp takes a head at a time and leaves the finished head in the staged row
    const int w = threadIdx.x >> 5, l = threadIdx.x & 31, ws = blockDim.x >> 5;
    for (int h = w; h < q_heads + kv_heads; h += ws) {
      float* head = row_s + (size_t)h * dim;
      const float* gain = h < q_heads ? q_gain : k_gain;
      float sq = 0.f;
      for (int d = l; d < dim; d += 32) sq = fmaf(head[d], head[d], sq);
      const float inv = rsqrtf(warp_sum(sq) / (float)dim + eps);
      for (int d = l; d < dim; d += 32) head[d] = gain[d] * (head[d] * inv);
    }
    __syncthreads();
  }
  const int pos = positions[t];
  if (inv_freq) {
    // a thread a pair: both elements are read before either is written, and no two pairs share an element
    const int half = rot_dims / 2;
    for (int e = threadIdx.x; e < (q_heads + kv_heads) * half; e += blockDim.x) {
      const int h = e / half, i = e % half;
      float* head = row_s + (size_t)h * dim;
      const int a = interleaved ? 2 * i : i, b = interleaved ? 2 * i + 1 : i + half;
      float sn, cs;
      sincosf((float)pos * inv_freq[i], &sn, &cs);
      sn *= magnitude;
      cs *= magnitude;
      const float u = head[a], v = head[b];
      head[a] = u * cs - v * sn;
      head[b] = v * cs + u * sn;
    }
    __syncthreads();
  }
  T* q_row = q_out + (size_t)t * q_stride;
  for (int i = threadIdx.x; i < q_width; i += blockDim.x) q_row[i] = from_float<T>(row_s[i]);
  if (!write_cache) return;
  const int request = request_of_token[t];
  const int index = pos / page_size;
  const int page = index < table_width ? table[(size_t)request * table_width + index] : -1;
  if (page < 0 || page >= num_pages) {
    if (threadIdx.x == 0) atomicOr(err, kErrBadPage);
    return;
  }
  const size_t slot = (size_t)page * kv_heads * page_size + (size_t)(pos % page_size);   // + head * page_size
  const float* k_row = row_s + q_width;
  for (int i = threadIdx.x; i < k_width; i += blockDim.x) {
    const int h = i / dim, d = i % dim;
    k_pool[(slot + (size_t)h * page_size) * dim + d] = from_float<T>(k_row[i]);
  }
  // value heads: a warp per head at a time
  const float* v_row = k_row + k_width;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
  for (int h = warp; h < kv_heads; h += warps) {
    float inv = 1.f;
    if (v_norm) {
      float sq = 0.f;
      for (int d = lane; d < vdim; d += 32) sq = fmaf(v_row[h * vdim + d], v_row[h * vdim + d], sq);
      inv = rsqrtf(warp_sum(sq) / (float)vdim + eps);
    }
    for (int d = lane; d < vdim; d += 32)
      v_pool[(slot + (size_t)h * page_size) * vdim + d] = from_float<T>(v_row[h * vdim + d] * inv);
  }
}

}  // namespace cie

using namespace cie;

#define DISPATCH_DTYPE(dtype, name, ...)                                   \
  if (dtype == kFloat32) { using T = float; __VA_ARGS__ }                 \
  else if (dtype == kBFloat16) { using T = __nv_bfloat16; __VA_ARGS__ }   \
  else CIE_FAIL("%s: unknown element type code %d", name, dtype);

static int threads_for(int n) {
  int t = 32;
  while (t < n && t < 1024) t <<= 1;
  return t;
}

template <typename K>
static int allow_shared(K kernel, size_t bytes, const char* name) {
  if (bytes > 200 * 1024) CIE_FAIL("%s: a row of %zu bytes does not fit shared memory", name, bytes);
  if (bytes > 48 * 1024 &&
      cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes) != cudaSuccess)
    CIE_FAIL("%s: cannot reserve %zu bytes of shared memory", name, bytes);
  return 0;
}

// residual: float32 [tokens][streams][hidden]; position_table may be null (then positions too).
extern "C" int cie_embedding_streams(const int* ids, const int* positions, const void* table,
                                     const void* position_table, float* residual, int tokens, int hidden,
                                     int vocab, int max_positions, int streams, float scale, int dtype,
                                     int* err, void* stream) {
  if (tokens <= 0) return 0;
  if (streams < 1) CIE_FAIL("embedding: %d streams", streams);
  DISPATCH_DTYPE(dtype, "embedding", {
    CIE_LAUNCH("embedding", embedding_streams_kernel<T>, dim3(tokens), dim3(threads_for(hidden / 4)), 0,
               (cudaStream_t)stream, ids, positions, (const T*)table, (const T*)position_table, residual,
               hidden, vocab, max_positions, streams, scale, err);
  })
  return 0;
}

// update_dtype: element type of `update` (float32, or the activation type `dtype`).
extern "C" int cie_stream_norm(float* streams, int num_streams, const void* update, int update_dtype,
                               const float* mix, const float* out_w, const float* read,
                               const float* gain, int gain_single, void* out, const int* rows, int count,
                               int hidden, float eps, int dtype, void* stream) {
  if (count <= 0) return 0;
  if (num_streams < 1 || num_streams > kMaxStreams) CIE_FAIL("stream_norm: 1..%d streams, got %d", kMaxStreams, num_streams);
  if (update && update_dtype != kFloat32 && update_dtype != dtype) CIE_FAIL("stream_norm: the update is float32 or of the activation type");
  const size_t smem = (size_t)hidden * sizeof(float);
  int threads = threads_for(hidden / 4);
  threads = threads < 64 ? 64 : (threads > 256 ? 256 : threads);
#define CIE_STREAM_NORM(T, TU, MAXS)                                                                          \
  do {                                                                                                         \
    if (allow_shared(stream_norm_kernel<T, TU, MAXS>, smem, "stream_norm")) return 1;                          \
    CIE_LAUNCH("stream_norm", (stream_norm_kernel<T, TU, MAXS>), dim3(count), dim3(threads), smem,             \
               (cudaStream_t)stream, streams, num_streams, (const TU*)update, mix, out_w, read, gain,          \
               gain_single, (T*)out, rows, hidden, eps);                                                       \
  } while (0)
  // up to four streams (the usual few) run an instance whose loops are unrolled to four
  DISPATCH_DTYPE(dtype, "stream_norm", {
    if (update_dtype == kFloat32) {
      if (num_streams <= 4) CIE_STREAM_NORM(T, float, 4);
      else CIE_STREAM_NORM(T, float, kMaxStreams);
    } else {
      if (num_streams <= 4) CIE_STREAM_NORM(T, T, 4);
      else CIE_STREAM_NORM(T, T, kMaxStreams);
    }
  })
#undef CIE_STREAM_NORM
  return 0;
}

extern "C" int cie_norm_kv_write(const void* src, const float* bias, void* q_out, int q_stride,
                                 const int* positions, const int* request_of_token, const int* table,
                                 int table_width, int num_pages, void* k_pool, void* v_pool,
                                 const float* q_gain, const float* k_gain, int tokens, int q_heads,
                                 int kv_heads, int dim, int vdim, int page_size, int qk_norm, int v_norm,
                                 float eps, int write_cache, int src_stride, int src_dtype,
                                 const float* inv_freq, int rot_dims, float magnitude, int interleaved,
                                 int dtype, int* err, void* stream) {
  // qk_norm: 0 none; 1 over the whole projection (gains of the projection's size); 2 per head (gains of a
  // head's size, shared by the heads).  src_stride: elements from one source row to the next (0: the
  // row holds q, k and v and nothing else).  src_dtype: float32 or the activation type `dtype`.
  if (tokens <= 0) return 0;
  if (qk_norm && (!q_gain || !k_gain)) CIE_FAIL("norm_kv_write: the q/k norm needs its gains");
  if (qk_norm < 0 || qk_norm > 2) CIE_FAIL("norm_kv_write: unknown q/k norm %d", qk_norm);
  if (inv_freq && (rot_dims < 2 || rot_dims % 2 || rot_dims > dim))
    CIE_FAIL("norm_kv_write: %d rotated elements of a head of %d", rot_dims, dim);
  if (src_dtype != kFloat32 && src_dtype != dtype) CIE_FAIL("norm_kv_write: the source is float32 or of the activation type");
  const int width = q_heads * dim + kv_heads * (dim + vdim);
  if (src_stride == 0) src_stride = width;
  if (src_stride < width) CIE_FAIL("norm_kv_write: source rows of %d elements are shorter than q, k and v (%d)", src_stride, width);
  const size_t smem = (size_t)width * sizeof(float);
#define CIE_NORM_KV(TI, T)                                                                                      \
  do {                                                                                                           \
    if (allow_shared(norm_kv_write_kernel<TI, T>, smem, "norm_kv_write")) return 1;                              \
    CIE_LAUNCH("norm_kv_write", (norm_kv_write_kernel<TI, T>), dim3(tokens), dim3(256), smem, (cudaStream_t)stream, \
               (const TI*)src, bias, (T*)q_out, q_stride, positions, request_of_token, table, table_width,       \
               num_pages, (T*)k_pool, (T*)v_pool, q_gain, k_gain, q_heads, kv_heads, dim, vdim, page_size,       \
               qk_norm, v_norm, eps, write_cache, src_stride, inv_freq, rot_dims, magnitude, interleaved, err);  \
  } while (0)
  DISPATCH_DTYPE(dtype, "norm_kv_write", {
    if (src_dtype == kFloat32) CIE_NORM_KV(float, T);
    else CIE_NORM_KV(T, T);
  })
#undef CIE_NORM_KV
  return 0;
}
