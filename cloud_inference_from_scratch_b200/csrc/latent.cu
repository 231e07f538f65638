// Attention over a cached latent ("latent attention"): what a token leaves in the pages is one
// normalised latent vector c [rank] and one rotated key part kr [rot] shared by all heads; keys and
// values of every head are linear maps of c.  Because the maps are linear the kernels below never
// expand keys or values:
//
//     score(t, h, j) = scale * ( (W_uk[h]^T q_plain[t,h]) . c_j + rotate(q_rot[t,h]) . kr_j )
//     out(t, h)      = W_uv[h] * sum_j weight(t,h,j) c_j
//
// so that attention is one-key-head attention over rows [c_j | kr_j] for all heads of a token, and
// the two maps are products per head before and after it (`head_linear`).
//
//   latent_prepare     per token: RMS norm of the query latent; RMS norm of c and rotation of kr,
//                      written into the pages
//   head_linear        out[t,h,:] = W[h]^T-laid-out product of x[t,h,:], optionally times sigmoid(gate)
//   latent_attention   softmax attention of every (token, head) over its request's rows, with an
//                      optional sink term in the denominator; keys cut into ranges over CTAs
//   latent_merge       joins the ranges
//
// Scores, softmax weights, norms, angles and the latent sums are float32 in both number formats;
// the pages hold the compute dtype.  A token's result depends on its own request's rows only.
#include "common.cuh"

#include <cfloat>

CIE_DEFINE_LAST_ERROR()

namespace cie {

// Pair (u, v) of a rotated vector: "half" pairs element i with i + dims/2, "interleaved" 2i with 2i+1.
__device__ __forceinline__ void pair_places(int i, int dims, int interleaved, int* a, int* b) {
  if (interleaved) { *a = 2 * i; *b = 2 * i + 1; } else { *a = i; *b = i + dims / 2; }
}

// ---------------------------------------------------------------- norms, rotation, cache write
// down: float32 [T, stride]: [query latent (q_rank) | latent (rank) | key part (rot)]; the last two
// only if has_kv.  q_out: [T, q_rank] in the compute dtype.
template <typename T>
__global__ void __launch_bounds__(128)
latent_prepare_kernel(const float* __restrict__ down, int stride, T* __restrict__ q_out,
                      const float* __restrict__ q_gain, const float* __restrict__ kv_gain,
                      const int* __restrict__ positions, const int* __restrict__ request_of_token,
                      const int* __restrict__ table, int table_width, int num_pages, T* __restrict__ c_pool,
                      T* __restrict__ r_pool, const float* __restrict__ inv_freq, float magnitude, int interleaved,
                      int rot_dims, int q_rank, int rank, int rot, int page_size, float eps, int has_kv,
                      int write_cache, int* err) {
  __shared__ float scratch[33];
  pdl_wait();
  pdl_trigger();
  const int t = blockIdx.x;
  const float* row = down + (size_t)t * stride;
  if (q_rank > 0) {
    float sq = 0.f;
    for (int i = threadIdx.x; i < q_rank; i += blockDim.x) sq += row[i] * row[i];
    const float inv = rsqrtf(block_sum(sq, scratch) / (float)q_rank + eps);
    for (int i = threadIdx.x; i < q_rank; i += blockDim.x)
      q_out[(size_t)t * q_rank + i] = from_float<T>(q_gain[i] * (row[i] * inv));
  }
  if (!has_kv || !write_cache) return;
  const float* kv = row + q_rank;
  float sq = 0.f;
  for (int i = threadIdx.x; i < rank; i += blockDim.x) sq += kv[i] * kv[i];
  const float inv = rsqrtf(block_sum(sq, scratch) / (float)rank + eps);
  const int pos = positions[t];
  const int page = table[(size_t)request_of_token[t] * table_width + pos / page_size];
  if (page < 0 || page >= num_pages) {
    if (threadIdx.x == 0) atomicOr(err, kErrBadPage);
    return;
  }
  const size_t slot = (size_t)page * page_size + pos % page_size;
  for (int i = threadIdx.x; i < rank; i += blockDim.x)
    c_pool[slot * rank + i] = from_float<T>(kv_gain[i] * (kv[i] * inv));
  const float* kr = kv + rank;
  T* dst = r_pool + slot * rot;
  for (int i = threadIdx.x; i < rot_dims / 2; i += blockDim.x) {
    int a, b;
    pair_places(i, rot_dims, interleaved, &a, &b);
    float s, c;
    sincosf((float)pos * inv_freq[i], &s, &c);
    s *= magnitude;
    c *= magnitude;
    const float u = kr[a], v = kr[b];
    dst[a] = from_float<T>(u * c - v * s);
    dst[b] = from_float<T>(v * c + u * s);
  }
  for (int i = rot_dims + threadIdx.x; i < rot; i += blockDim.x) dst[i] = from_float<T>(kr[i]);
}

// ---------------------------------------------------------------- products per head
// out[t, h, j] = sum_k x[t, h, k] * w[h][k][j]   (k ascending, one fused multiply-add each)
// x: float32, element (t, h, k) at x[t * x_stride + h * x_head + k]; w: [heads, K, N] in the compute
// dtype; out element at out[t * out_stride + h * out_head + j], float32 or the compute dtype.
// gate != nullptr: the result is multiplied by sigmoid(gate[t * gate_stride + h * N + j]).
constexpr int kHeadTokens = 16;     // tokens of a block
constexpr int kHeadColumns = 128;   // output columns of a block: one per thread
constexpr int kHeadChunk = 64;      // k values staged at a time

template <typename TW, typename TO>
__global__ void __launch_bounds__(kHeadColumns)
head_linear_kernel(const float* __restrict__ x, int x_stride, int x_head, const TW* __restrict__ w,
                   TO* __restrict__ out, int out_stride, int out_head, const float* __restrict__ gate,
                   int gate_stride, int tokens, int K, int N) {
  __shared__ __align__(16) float xs[kHeadChunk][kHeadTokens];
  pdl_wait();
  pdl_trigger();
  const int t0 = blockIdx.x * kHeadTokens, h = blockIdx.y;
  const int j = blockIdx.z * kHeadColumns + threadIdx.x;
  const int count = min(kHeadTokens, tokens - t0);
  const TW* wh = w + (size_t)h * K * N;
  float acc[kHeadTokens];
#pragma unroll
  for (int i = 0; i < kHeadTokens; ++i) acc[i] = 0.f;
  for (int k0 = 0; k0 < K; k0 += kHeadChunk) {
    const int kn = min(kHeadChunk, K - k0);
    __syncthreads();
    for (int e = threadIdx.x; e < kHeadChunk * kHeadTokens; e += blockDim.x) {
      const int i = e / kHeadChunk, k = e % kHeadChunk;
      xs[k][i] = (i < count && k < kn) ? x[(size_t)(t0 + i) * x_stride + (size_t)h * x_head + k0 + k] : 0.f;
    }
    __syncthreads();
    if (j < N) {
      for (int k = 0; k < kn; ++k) {
        const float wv = to_float(wh[(size_t)(k0 + k) * N + j]);
        const float4* xv = reinterpret_cast<const float4*>(xs[k]);
#pragma unroll
        for (int i = 0; i < kHeadTokens / 4; ++i) {
          const float4 v = xv[i];
          acc[4 * i] = fmaf(v.x, wv, acc[4 * i]);
          acc[4 * i + 1] = fmaf(v.y, wv, acc[4 * i + 1]);
          acc[4 * i + 2] = fmaf(v.z, wv, acc[4 * i + 2]);
          acc[4 * i + 3] = fmaf(v.w, wv, acc[4 * i + 3]);
        }
      }
    }
  }
  if (j >= N) return;
#pragma unroll
  for (int i = 0; i < kHeadTokens; ++i) {
    if (i < count) {
      float v = acc[i];
      if (gate) v *= 1.f / (1.f + expf(-gate[(size_t)(t0 + i) * gate_stride + (size_t)h * N + j]));
      out[(size_t)(t0 + i) * out_stride + (size_t)h * out_head + j] = from_float<TO>(v);
    }
  }
}

// The same product for at most kHeadTokens tokens (a decode step): what bounds it is the walk over K, so K
// is cut into kFewSlices slices over the warps of a block, a block takes 32 columns of one head, and the
// slices meet in shared memory and are added in ascending order.
constexpr int kFewSlices = 8;
constexpr int kFewColumns = 32;
constexpr int kFewMaxK = 256;      // rows of x staged at a time

template <typename TW, typename TO>
__global__ void __launch_bounds__(kFewSlices * kFewColumns)
head_linear_few_kernel(const float* __restrict__ x, int x_stride, int x_head, const TW* __restrict__ w,
                       TO* __restrict__ out, int out_stride, int out_head, const float* __restrict__ gate,
                       int gate_stride, int tokens, int K, int N) {
  __shared__ __align__(16) float xs[kFewMaxK][kHeadTokens];                 // 16 KB
  __shared__ float sums[kFewSlices][kHeadTokens][kFewColumns + 1];
  pdl_wait();
  pdl_trigger();
  const int h = blockIdx.x;
  const int slice = threadIdx.x / kFewColumns, lane = threadIdx.x % kFewColumns;
  const int j = blockIdx.y * kFewColumns + lane;
  const TW* wh = w + (size_t)h * K * N;
  float acc[kHeadTokens];
#pragma unroll
  for (int i = 0; i < kHeadTokens; ++i) acc[i] = 0.f;
  for (int k0 = 0; k0 < K; k0 += kFewMaxK) {
    const int kn = min(kFewMaxK, K - k0);
    __syncthreads();
    for (int e = threadIdx.x; e < kn * kHeadTokens; e += blockDim.x) {
      const int i = e / kn, k = e % kn;
      xs[k][i] = i < tokens ? x[(size_t)i * x_stride + (size_t)h * x_head + k0 + k] : 0.f;
    }
    __syncthreads();
    if (j < N) {
#pragma unroll 4
      for (int k = slice; k < kn; k += kFewSlices) {
        const float wv = to_float(wh[(size_t)(k0 + k) * N + j]);
        const float4* xv = reinterpret_cast<const float4*>(xs[k]);
#pragma unroll
        for (int i = 0; i < kHeadTokens / 4; ++i) {
          const float4 v = xv[i];
          acc[4 * i] = fmaf(v.x, wv, acc[4 * i]);
          acc[4 * i + 1] = fmaf(v.y, wv, acc[4 * i + 1]);
          acc[4 * i + 2] = fmaf(v.z, wv, acc[4 * i + 2]);
          acc[4 * i + 3] = fmaf(v.w, wv, acc[4 * i + 3]);
        }
      }
    }
  }
#pragma unroll
  for (int i = 0; i < kHeadTokens; ++i) sums[slice][i][lane] = acc[i];
  __syncthreads();
  for (int e = threadIdx.x; e < tokens * kFewColumns; e += blockDim.x) {
    const int i = e / kFewColumns, c = e % kFewColumns;
    const int column = blockIdx.y * kFewColumns + c;
    if (column >= N) continue;
    float v = 0.f;
#pragma unroll
    for (int sl = 0; sl < kFewSlices; ++sl) v += sums[sl][i][c];
    if (gate) v *= 1.f / (1.f + expf(-gate[(size_t)i * gate_stride + (size_t)h * N + column]));
    out[(size_t)i * out_stride + (size_t)h * out_head + column] = from_float<TO>(v);
  }
}

// For many tokens the products per head run as one batched library product over [heads, T, K] x
// [heads, K, N]; these two kernels carry the rows there and back.
// gather: dst[h][t][k] = bfloat16(x[t * x_stride + h * x_head + k])
__global__ void head_gather_kernel(const float* __restrict__ x, int x_stride, int x_head, __nv_bfloat16* __restrict__ dst,
                                   int tokens, int heads, int K) {
  pdl_wait();
  pdl_trigger();
  const size_t total = (size_t)tokens * heads * K;
  for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (size_t)gridDim.x * blockDim.x) {
    const int k = (int)(e % K);
    const size_t th = e / K;
    const int h = (int)(th % heads);
    const size_t t = th / heads;
    dst[((size_t)h * tokens + t) * K + k] = __float2bfloat16_rn(x[t * x_stride + (size_t)h * x_head + k]);
  }
}

// scatter: out[t * out_stride + h * out_head + j] = y[h][t][j] (* sigmoid(gate[t * gate_stride + h * N + j]))
template <typename TO>
__global__ void head_scatter_kernel(const __nv_bfloat16* __restrict__ y, TO* __restrict__ out, int out_stride, int out_head,
                                    const float* __restrict__ gate, int gate_stride, int tokens, int heads, int N) {
  pdl_wait();
  pdl_trigger();
  const size_t total = (size_t)tokens * heads * N;
  for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (size_t)gridDim.x * blockDim.x) {
    const int j = (int)(e % N);
    const size_t th = e / N;
    const int h = (int)(th % heads);
    const size_t t = th / heads;
    float v = __bfloat162float(y[((size_t)h * tokens + t) * N + j]);
    if (gate) v *= 1.f / (1.f + expf(-gate[t * gate_stride + (size_t)h * N + j]));
    out[t * out_stride + (size_t)h * out_head + j] = from_float<TO>(v);
  }
}

// ---------------------------------------------------------------- attention
// One CTA per (token, group of kAttnHeads heads, key range); a warp per head.  The rows
// [c_j | kr_j] of 32 keys at a time are staged in shared memory as float32 and shared by the warps:
// for the scores a lane owns a key, for the sums a lane owns latent columns.  Keys are visited in
// blocks of 32 counted from the start of the CTA's range, ranges are `range_keys` long counted from
// key 0, so a token's result depends on nothing but its own request's rows and `range_keys`.
//
// q_abs: float32 [T, heads, rank] (the plain query part mapped into the latent); q_raw: float32,
// element (t, h, d) of the rotated part at q_raw[t * q_raw_stride + h * q_raw_head + d], not yet
// rotated.  ranges == 1: the normalised sum goes to out [T, heads, rank]; else the CTA leaves
// (maximum, sum, unnormalised latent sum) in part [T, heads, ranges, rank + 2].
constexpr int kAttnHeads = 8;
constexpr int kLatentMaxRank = 1024;

__host__ __device__ __forceinline__ size_t latent_row_floats(int rank, int rot) { return (size_t)((rank + rot) | 1); }

template <typename T>
__global__ void __launch_bounds__(kAttnHeads * 32)
latent_attention_kernel(const float* __restrict__ q_abs, const float* __restrict__ q_raw, int q_raw_stride,
                        int q_raw_head, float* __restrict__ out, float* __restrict__ part,
                        const T* __restrict__ c_pool, const T* __restrict__ r_pool,
                        const int* __restrict__ positions, const int* __restrict__ request_of_token,
                        const int* __restrict__ table, int table_width, int num_pages,
                        const float* __restrict__ inv_freq, float magnitude, int interleaved, int rot_dims,
                        const float* __restrict__ sink, int heads, int rank, int rot, int page_size, float scale,
                        int range_keys, int ranges, int window, int* err) {
  extern __shared__ __align__(16) float shared[];
  const int D = rank + rot;
  const int ld = (int)latent_row_floats(rank, rot);
  float* ks = shared;                                   // [32][ld]
  float* qs = ks + 32 * ld;                             // [kAttnHeads][D]
  float* ps = qs + kAttnHeads * D;                      // [kAttnHeads][32]
  __shared__ long long row_of[32];
  pdl_wait();
  pdl_trigger();
  const int t = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int h = blockIdx.y * kAttnHeads + warp;
  const bool live = h < heads;
  const int pos = positions[t];
  const int length = pos + 1;
  // window > 0: the token sees its last `window` keys (itself included); ranges count from the first of them
  const int first = (window > 0 && length > window) ? length - window : 0;
  const int begin = first + blockIdx.z * range_keys;
  if (begin >= length) return;
  const int end = min(length, begin + range_keys);
  const int* pages = table + (size_t)request_of_token[t] * table_width;

  if (live) {
    const float* qa = q_abs + ((size_t)t * heads + h) * rank;
    for (int d = lane; d < rank; d += 32) qs[warp * D + d] = qa[d];
    const float* qr = q_raw + (size_t)t * q_raw_stride + (size_t)h * q_raw_head;
    for (int i = lane; i < rot_dims / 2; i += 32) {
      int a, b;
      pair_places(i, rot_dims, interleaved, &a, &b);
      float s, c;
      sincosf((float)pos * inv_freq[i], &s, &c);
      s *= magnitude;
      c *= magnitude;
      const float u = qr[a], v = qr[b];
      qs[warp * D + rank + a] = u * c - v * s;
      qs[warp * D + rank + b] = v * c + u * s;
    }
    for (int i = rot_dims + lane; i < rot; i += 32) qs[warp * D + rank + i] = qr[i];
  }

  constexpr int kMaxCols = kLatentMaxRank / 32;         // latent columns of a lane
  float acc[kMaxCols];
#pragma unroll
  for (int i = 0; i < kMaxCols; ++i) acc[i] = 0.f;
  float m = -FLT_MAX, l = 0.f;

  for (int base = begin; base < end; base += 32) {
    const int n = min(32, end - base);
    __syncthreads();                                    // the tile before this one has been read
    if (threadIdx.x < 32) {
      long long r = -1;
      if (threadIdx.x < n) {
        const int key = base + threadIdx.x;
        const int page = pages[key / page_size];
        if (page < 0 || page >= num_pages) atomicOr(err, kErrBadPage);
        else r = (long long)page * page_size + key % page_size;
      }
      row_of[threadIdx.x] = r;
    }
    __syncthreads();
    for (int e = threadIdx.x; e < 32 * D; e += blockDim.x) {
      const int j = e / D, d = e % D;
      const long long r = row_of[j];
      float v = 0.f;
      if (r >= 0) v = d < rank ? to_float(c_pool[(size_t)r * rank + d]) : to_float(r_pool[(size_t)r * rot + d - rank]);
      ks[j * ld + d] = v;
    }
    __syncthreads();
    if (!live) continue;
    const float* q = qs + warp * D;
    const float* k = ks + lane * ld;
    float s = 0.f;
    for (int d = 0; d < D; ++d) s = fmaf(q[d], k[d], s);
    s = lane < n ? s * scale : -FLT_MAX;
    const float m_new = fmaxf(m, warp_max(s));
    const float p = lane < n ? expf(s - m_new) : 0.f;
    const float fix = expf(m - m_new);
    l = l * fix + warp_sum(p);
    m = m_new;
    ps[warp * 32 + lane] = p;
    __syncwarp();
#pragma unroll
    for (int i = 0; i < kMaxCols; ++i) {
      const int col = lane + 32 * i;
      if (col < rank) {
        float a = acc[i] * fix;
        for (int j = 0; j < n; ++j) a = fmaf(ps[warp * 32 + j], ks[j * ld + col], a);
        acc[i] = a;
      }
    }
    __syncwarp();
  }
  if (!live) return;
  if (ranges == 1) {
    float total = l;
    float keep = 1.f;
    if (sink) {
      const float top = fmaxf(m, sink[h]);
      keep = expf(m - top);
      total = l * keep + expf(sink[h] - top);
    }
    const float inv = keep / total;
    float* o = out + ((size_t)t * heads + h) * rank;
#pragma unroll
    for (int i = 0; i < kMaxCols; ++i) {
      const int col = lane + 32 * i;
      if (col < rank) o[col] = acc[i] * inv;
    }
    return;
  }
  float* share = part + (((size_t)t * heads + h) * ranges + blockIdx.z) * (rank + 2);
  if (lane == 0) {
    share[0] = m;
    share[1] = l;
  }
#pragma unroll
  for (int i = 0; i < kMaxCols; ++i) {
    const int col = lane + 32 * i;
    if (col < rank) share[2 + col] = acc[i];
  }
}

// Joins the key ranges of every (token, head): grid (tokens, heads), in ascending range order.
__global__ void __launch_bounds__(128)
latent_merge_kernel(const float* __restrict__ part, float* __restrict__ out, const int* __restrict__ positions,
                    const float* __restrict__ sink, int heads, int rank, int range_keys, int ranges, int window) {
  constexpr int kHeld = 256;          // weights of this many ranges are worked out once and kept
  __shared__ float held[kHeld];
  pdl_wait();
  pdl_trigger();
  const int t = blockIdx.x, h = blockIdx.y;
  const int seen = window > 0 ? min(positions[t] + 1, window) : positions[t] + 1;      // visible keys
  const int used = min(ranges, (seen + range_keys - 1) / range_keys);
  const float* share = part + ((size_t)t * heads + h) * ranges * (rank + 2);
  float top = sink ? sink[h] : -FLT_MAX;
  for (int r = 0; r < used; ++r) top = fmaxf(top, share[(size_t)r * (rank + 2)]);
  for (int r = threadIdx.x; r < min(used, kHeld); r += blockDim.x) held[r] = expf(share[(size_t)r * (rank + 2)] - top);
  __syncthreads();
  auto weight = [&](int r) { return r < kHeld ? held[r] : expf(share[(size_t)r * (rank + 2)] - top); };
  float total = sink ? expf(sink[h] - top) : 0.f;
  for (int r = 0; r < used; ++r) total += share[(size_t)r * (rank + 2) + 1] * weight(r);
  const float inv = 1.f / total;
  for (int col = threadIdx.x; col < rank; col += blockDim.x) {
    float a = 0.f;
    for (int r = 0; r < used; ++r) a = fmaf(share[(size_t)r * (rank + 2) + 2 + col], weight(r), a);
    out[((size_t)t * heads + h) * rank + col] = a * inv;
  }
}

}  // namespace cie

#define DISPATCH_DTYPE(code, name, ...)                              \
  if ((code) == cie::kFloat32) { using T = float; __VA_ARGS__ }      \
  else if ((code) == cie::kBFloat16) { using T = __nv_bfloat16; __VA_ARGS__ } \
  else CIE_FAIL("%s: unknown dtype code %d", name, (code));

extern "C" int cie_latent_prepare(const float* down, int stride, void* q_out, const float* q_gain,
                                  const float* kv_gain, const int* positions, const int* request_of_token,
                                  const int* table, int table_width, int num_pages, void* c_pool, void* r_pool,
                                  const float* inv_freq, float magnitude, int interleaved, int rot_dims,
                                  int tokens, int q_rank, int rank, int rot, int page_size, float eps, int has_kv,
                                  int write_cache, int dtype, int* err, void* stream) {
  using namespace cie;
  if (tokens <= 0) return 0;
  if (rot_dims % 2 || rot_dims > rot) CIE_FAIL("latent_prepare: %d rotated dims of %d", rot_dims, rot);
  DISPATCH_DTYPE(dtype, "latent_prepare", {
    CIE_LAUNCH("latent_prepare", latent_prepare_kernel<T>, dim3(tokens), dim3(128), 0, (cudaStream_t)stream, down,
               stride, (T*)q_out, q_gain, kv_gain, positions, request_of_token, table, table_width, num_pages,
               (T*)c_pool, (T*)r_pool, inv_freq, magnitude, interleaved, rot_dims, q_rank, rank, rot, page_size,
               eps, has_kv, write_cache, err);
  })
  return 0;
}

extern "C" int cie_head_linear(const float* x, int x_stride, int x_head, const void* w, void* out,
                               int out_stride, int out_head, const float* gate, int gate_stride, int tokens,
                               int heads, int K, int N, int w_dtype, int out_dtype, void* stream) {
  using namespace cie;
  if (tokens <= 0 || heads <= 0 || N <= 0) return 0;
  const bool few = tokens <= kHeadTokens;
  const dim3 grid = few ? dim3(heads, (N + kFewColumns - 1) / kFewColumns)
                        : dim3((tokens + kHeadTokens - 1) / kHeadTokens, heads, (N + kHeadColumns - 1) / kHeadColumns);
  if (grid.y > 65535 || grid.z > 65535) CIE_FAIL("head_linear: too many heads or columns");
#define CIE_HEAD_LINEAR(TW, TO)                                                                                   \
  if (few) {                                                                                                      \
    CIE_LAUNCH("head_linear", (head_linear_few_kernel<TW, TO>), grid, dim3(kFewSlices * kFewColumns), 0,          \
               (cudaStream_t)stream, x, x_stride, x_head, (const TW*)w, (TO*)out, out_stride, out_head, gate,     \
               gate_stride, tokens, K, N);                                                                        \
  } else                                                                                                          \
    CIE_LAUNCH("head_linear", (head_linear_kernel<TW, TO>), grid, dim3(kHeadColumns), 0, (cudaStream_t)stream, x, \
               x_stride, x_head, (const TW*)w, (TO*)out, out_stride, out_head, gate, gate_stride, tokens, K, N)
  if (w_dtype == kFloat32 && out_dtype == kFloat32) { CIE_HEAD_LINEAR(float, float); }
  else if (w_dtype == kBFloat16 && out_dtype == kFloat32) { CIE_HEAD_LINEAR(__nv_bfloat16, float); }
  else if (w_dtype == kBFloat16 && out_dtype == kBFloat16) { CIE_HEAD_LINEAR(__nv_bfloat16, __nv_bfloat16); }
  else CIE_FAIL("head_linear: weight dtype %d with output dtype %d", w_dtype, out_dtype);
#undef CIE_HEAD_LINEAR
  return 0;
}

extern "C" int cie_head_gather(const float* x, int x_stride, int x_head, void* dst, int tokens, int heads, int K,
                               void* stream) {
  using namespace cie;
  const size_t total = (size_t)tokens * heads * K;
  if (total == 0) return 0;
  const int blocks = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
  CIE_LAUNCH("head_gather", head_gather_kernel, dim3(blocks), dim3(256), 0, (cudaStream_t)stream, x, x_stride, x_head,
             (__nv_bfloat16*)dst, tokens, heads, K);
  return 0;
}

extern "C" int cie_head_scatter(const void* y, void* out, int out_stride, int out_head, const float* gate,
                                int gate_stride, int tokens, int heads, int N, int out_dtype, void* stream) {
  using namespace cie;
  const size_t total = (size_t)tokens * heads * N;
  if (total == 0) return 0;
  const int blocks = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
  DISPATCH_DTYPE(out_dtype, "head_scatter", {
    CIE_LAUNCH("head_scatter", head_scatter_kernel<T>, dim3(blocks), dim3(256), 0, (cudaStream_t)stream,
               (const __nv_bfloat16*)y, (T*)out, out_stride, out_head, gate, gate_stride, tokens, heads, N);
  })
  return 0;
}

extern "C" int cie_latent_merge(const float* part, float* out, const int* positions, const float* sink, int tokens,
                                int heads, int rank, int range_keys, int ranges, int window, void* stream) {
  using namespace cie;
  if (tokens <= 0) return 0;
  CIE_LAUNCH("latent_merge", latent_merge_kernel, dim3(tokens, heads), dim3(128), 0, (cudaStream_t)stream, part, out,
             positions, sink, heads, rank, range_keys, ranges, window);
  return 0;
}

extern "C" int cie_latent_attention_max_rank() { return cie::kLatentMaxRank; }

extern "C" int cie_latent_attention(const float* q_abs, const float* q_raw, int q_raw_stride, int q_raw_head,
                                    float* out, float* part, const void* c_pool, const void* r_pool,
                                    const int* positions, const int* request_of_token, const int* table,
                                    int table_width, int num_pages, const float* inv_freq, float magnitude,
                                    int interleaved, int rot_dims, const float* sink, int tokens, int heads,
                                    int rank, int rot, int page_size, float scale, int range_keys, int ranges,
                                    int window, int dtype, int* err, void* stream) {
  using namespace cie;
  if (tokens <= 0) return 0;
  if (rank > kLatentMaxRank) CIE_FAIL("latent_attention: latent size %d is above %d", rank, kLatentMaxRank);
  if (range_keys < 32 || range_keys % 32) CIE_FAIL("latent_attention: key ranges are multiples of 32, got %d", range_keys);
  if (ranges < 1 || ranges > 65535) CIE_FAIL("latent_attention: %d key ranges", ranges);
  if (ranges > 1 && !part) CIE_FAIL("latent_attention: key ranges need scratch memory");
  const int D = rank + rot;
  const size_t smem = (32 * latent_row_floats(rank, rot) + (size_t)kAttnHeads * D + kAttnHeads * 32) * sizeof(float);
  const dim3 grid(tokens, (heads + kAttnHeads - 1) / kAttnHeads, ranges);
  DISPATCH_DTYPE(dtype, "latent_attention", {
    static bool raised = false;
    if (!raised) {
      if (cudaFuncSetAttribute(latent_attention_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) != cudaSuccess)
        CIE_FAIL("latent_attention: cannot raise the shared memory limit");
      raised = true;
    }
    if (smem > 200 * 1024) CIE_FAIL("latent_attention: rows of %d elements need %zu bytes of shared memory", D, smem);
    CIE_LAUNCH("latent_attention", latent_attention_kernel<T>, grid, dim3(kAttnHeads * 32), smem, (cudaStream_t)stream,
               q_abs, q_raw, q_raw_stride, q_raw_head, out, part, (const T*)c_pool, (const T*)r_pool, positions,
               request_of_token, table, table_width, num_pages, inv_freq, magnitude, interleaved, rot_dims, sink,
               heads, rank, rot, page_size, scale, range_keys, ranges, window, err);
  })
  if (ranges > 1)
    CIE_LAUNCH("latent_merge", latent_merge_kernel, dim3(tokens, heads), dim3(128), 0, (cudaStream_t)stream, part, out,
               positions, sink, heads, rank, range_keys, ranges, window);
  return 0;
}
