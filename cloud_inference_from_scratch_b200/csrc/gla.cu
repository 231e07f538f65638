// Gated linear attention: linear attention whose state decays by a factor of its own per key channel and token,
//
//     S_t = diag(alpha_t) S_(t-1) + k_t v_t^T          (S: [dim][vdim], float32, one per request and head)
//     o_t = S_t^T q_t,       alpha_t = sigmoid(z_t + bias)^(1 / tau)   (one number per head and key channel)
//
// over a ragged batch: every request brings one or more new tokens and continues from the state its slot holds.
// q, k and v arrive as columns of one float32 row per token (the projections' float32 results, never rounded
// again), z as a float32 row of its own [heads * dim]; q is multiplied by `q_scale` here.  The logarithm of the
// decay is log(alpha) = -softplus(-(z + bias)) / tau, worked out in float32; everything of the recurrence is
// float32 on the CUDA cores.
//
// Two forms.  `gla_scan_kernel` walks a request's tokens one by one (single tokens of a decode step, and key
// sizes above 128).  Prompt portions run in chunks of 32 tokens (key and value sizes up to 128): with
// b_i = sum_(s<=i) log(alpha_s) counted from the chunk's first token and S_0 the state before the chunk,
//
//     o_i = (q_i * exp(b_i))^T S_0 + sum_(j<=i) (sum_d q_i[d] k_j[d] exp(b_i[d] - b_j[d])) v_j
//     S_n = diag(exp(b_n)) S_0 + sum_j (k_j * exp(b_n - b_j)) v_j^T
//
// in which no exponent is above zero: (0) per (chunk, head) the sums b_i, left in the place of the decay logits;
// (1) per (chunk, head) the sum over j and exp(b_n); (2) per (request, head) a walk over the request's chunks
// that leaves the state BEFORE each chunk in the sum's place and the last state in the slot; (3) per (chunk,
// head) the outputs.  Chunks come as a work list made on the host from the step's
// portion lengths (first token row and token count of each chunk; where every request's chunks start).
//
// A request's result depends on its own tokens and state only: the batch and the slot change nothing, the cut
// of a prompt into portions only the order of additions.
#include "common.cuh"

CIE_DEFINE_LAST_ERROR()

namespace cie {

constexpr int kScanWarps = 8;        // warps of a block; in the scan warp w owns state rows w, w + 8, ...
constexpr int kScanColumns = 32;     // value columns of a scan block: one per lane
constexpr int kScanRows = 32;        // state rows a warp keeps in registers (dim <= 8 * 32)

// log(sigmoid(y)) / tau = -softplus(-y) / tau, without overflow for any y
__device__ __forceinline__ float log_decay(float y, float inv_tau) {
  return -(fmaxf(-y, 0.f) + log1pf(expf(-fabsf(y)))) * inv_tau;
}

struct GlaRows {
  const float* proj;     // [tokens][proj_stride]
  int proj_stride;
  int q_off, k_off, v_off;   // first column of q, k and v (heads side by side inside each)
  const float* z;        // [tokens][z_stride]: decay logits, heads x dim
  int z_stride;
  const float* z_bias;   // [heads * dim]
  float inv_tau;
  float q_scale;
};

// grid: (requests, heads, ceil(vdim / 32)).
__global__ void __launch_bounds__(kScanWarps * 32)
gla_scan_kernel(GlaRows in, float* __restrict__ out, int out_stride, float* __restrict__ state,
                const int* __restrict__ query_start, const int* __restrict__ slots,
                const int* __restrict__ request_active, int heads, int dim, int vdim, int max_slots, int* err) {
  __shared__ float q_s[2][kScanWarps * kScanRows], k_s[2][kScanWarps * kScanRows], a_s[2][kScanWarps * kScanRows];
  __shared__ float part_s[2][kScanWarps][kScanColumns];
  pdl_wait();
  pdl_trigger();
  const int request = blockIdx.x, head = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int column = blockIdx.z * kScanColumns + lane;
  const bool live = column < vdim;
  const int slot = slots[request];
  if (slot < 0 || slot >= max_slots) {
    if (threadIdx.x == 0) atomicOr(err, kErrBadRequest);
    return;
  }
  const int begin = query_start[request], end = query_start[request + 1];
  float* s_base = state + (((size_t)slot * heads + head) * dim) * vdim;
  float s[kScanRows];
#pragma unroll
  for (int r = 0; r < kScanRows; ++r) {
    const int i = warp + kScanWarps * r;
    s[r] = (i < dim && live) ? s_base[(size_t)i * vdim + column] : 0.f;
  }
  for (int t = begin; t < end; ++t) {
    const int buf = (t - begin) & 1;
    const float* row = in.proj + (size_t)t * in.proj_stride;
    const float* zr = in.z + (size_t)t * in.z_stride + head * dim;
    for (int i = threadIdx.x; i < dim; i += blockDim.x) {
      q_s[buf][i] = row[in.q_off + head * dim + i] * in.q_scale;
      k_s[buf][i] = row[in.k_off + head * dim + i];
      a_s[buf][i] = expf(log_decay(zr[i] + in.z_bias[head * dim + i], in.inv_tau));
    }
    const float v = live ? row[in.v_off + head * vdim + column] : 0.f;
    __syncthreads();
    float o = 0.f;
#pragma unroll
    for (int r = 0; r < kScanRows; ++r) {
      const int i = warp + kScanWarps * r;
      if (i < dim) {
        s[r] = fmaf(a_s[buf][i], s[r], k_s[buf][i] * v);
        o = fmaf(s[r], q_s[buf][i], o);
      }
    }
    part_s[buf][warp][lane] = o;
    __syncthreads();
    if (warp == 0 && live) {
      float total = 0.f;
#pragma unroll
      for (int w = 0; w < kScanWarps; ++w) total += part_s[buf][w][lane];
      out[(size_t)t * out_stride + head * vdim + column] = total;
    }
    // the buffers of token t are read again only after the first barrier of token t + 2
  }
  if (request_active[request] && live) {
#pragma unroll
    for (int r = 0; r < kScanRows; ++r) {
      const int i = warp + kScanWarps * r;
      if (i < dim) s_base[(size_t)i * vdim + column] = s[r];
    }
  }
}

// ---------------------------------------------------------------- prompt portions in chunks
constexpr int kChunk = 32;
constexpr int kChunkDim = 128;                          // largest key and value size of the chunked kernels
constexpr int kChunkRows = kChunkDim / kScanWarps;      // state rows of a warp
constexpr int kChunkCols = kChunkDim / 32;              // value columns of a lane

// dst[j * ld + i] = src[row0 + j][col0 + i] * factor for j < n, i < width
__device__ __forceinline__ void stage_rows(float* __restrict__ dst, int ld, const float* __restrict__ src, int stride,
                                           int row0, int n, int col0, int width, float factor) {
  if (width % 4 == 0 && col0 % 4 == 0 && stride % 4 == 0 && ld % 4 == 0 && (reinterpret_cast<uintptr_t>(src) & 15) == 0) {
    const int pieces = width / 4;
    for (int e = threadIdx.x; e < n * pieces; e += blockDim.x) {
      const int j = e / pieces, i = (e % pieces) * 4;
      float4 v = *reinterpret_cast<const float4*>(src + (size_t)(row0 + j) * stride + col0 + i);
      v.x *= factor; v.y *= factor; v.z *= factor; v.w *= factor;
      *reinterpret_cast<float4*>(dst + j * ld + i) = v;
    }
    return;
  }
  for (int e = threadIdx.x; e < n * width; e += blockDim.x) {
    const int j = e / width, i = e % width;
    dst[j * ld + i] = src[(size_t)(row0 + j) * stride + col0 + i] * factor;
  }
}

// (0) z[row0 + j][head][d] <- b_j[d] = sum_(s<=j) log(alpha_s[d]) for the chunk's tokens j < n, in place: a thread a
// channel adds the logarithms up in token order.  Both kernels that follow read the sums from there.
__global__ void gla_decay_sums_kernel(float* __restrict__ z, int z_stride, const float* __restrict__ z_bias,
                                      float inv_tau, const int* __restrict__ chunk_row,
                                      const int* __restrict__ chunk_count, int dim) {
  pdl_wait();
  pdl_trigger();
  const int chunk = blockIdx.x, head = blockIdx.y;
  const int row0 = chunk_row[chunk], n = chunk_count[chunk];
  for (int d = threadIdx.x; d < dim; d += blockDim.x) {
    float* cell = z + (size_t)row0 * z_stride + head * dim + d;
    const float bias = z_bias[head * dim + d];
    float sum = 0.f;
    for (int j0 = 0; j0 < n; j0 += 8) {        // eight loads in flight, then their logarithms in token order
      float y[8];
#pragma unroll
      for (int x = 0; x < 8; ++x) y[x] = j0 + x < n ? cell[(size_t)(j0 + x) * z_stride] : 0.f;
#pragma unroll
      for (int x = 0; x < 8; ++x) {
        if (j0 + x < n) {
          sum += log_decay(y[x] + bias, inv_tau);
          cell[(size_t)(j0 + x) * z_stride] = sum;
        }
      }
    }
  }
}

// (1) chunk_state[chunk][head] = sum_j (k_j * exp(b_n - b_j)) v_j^T; chunk_decay[chunk][head][d] = exp(b_n[d]).
__global__ void __launch_bounds__(kScanWarps * 32)
gla_chunk_state_kernel(GlaRows in, float* __restrict__ chunk_state, float* __restrict__ chunk_decay,
                       const int* __restrict__ chunk_row, const int* __restrict__ chunk_count, int heads, int dim,
                       int vdim) {
  extern __shared__ __align__(16) float smem[];
  float* k_s = smem;                          // [kChunk][dim], times exp(b_n - b_j)
  float* v_s = k_s + kChunk * dim;            // [kChunk][vdim]
  pdl_wait();
  pdl_trigger();
  const int chunk = blockIdx.x, head = blockIdx.y;
  const int row0 = chunk_row[chunk], n = chunk_count[chunk];
  stage_rows(v_s, vdim, in.proj, in.proj_stride, row0, n, in.v_off + head * vdim, vdim, 1.f);
  const float* b_last = in.z + (size_t)(row0 + n - 1) * in.z_stride + head * dim;
  const int k_col = in.k_off + head * dim;
  if (dim % 4 == 0 && k_col % 4 == 0 && in.proj_stride % 4 == 0 && in.z_stride % 4 == 0 &&
      ((reinterpret_cast<uintptr_t>(in.proj) | reinterpret_cast<uintptr_t>(in.z)) & 15) == 0) {
    // 16-byte pieces of the key rows and of the sums (one index division a piece)
    const int pieces = dim / 4;
    for (int e = threadIdx.x; e < n * pieces; e += blockDim.x) {
      const int j = e / pieces, d = (e % pieces) * 4;
      const float4 b = *reinterpret_cast<const float4*>(in.z + (size_t)(row0 + j) * in.z_stride + head * dim + d);
      const float4 last = *reinterpret_cast<const float4*>(b_last + d);
      float4 k = *reinterpret_cast<const float4*>(in.proj + (size_t)(row0 + j) * in.proj_stride + k_col + d);
      k.x *= expf(last.x - b.x); k.y *= expf(last.y - b.y); k.z *= expf(last.z - b.z); k.w *= expf(last.w - b.w);
      *reinterpret_cast<float4*>(k_s + j * dim + d) = k;
    }
  } else {
    for (int e = threadIdx.x; e < n * dim; e += blockDim.x) {
      const int j = e / dim, d = e % dim;
      const float b = in.z[(size_t)(row0 + j) * in.z_stride + head * dim + d];
      k_s[e] = in.proj[(size_t)(row0 + j) * in.proj_stride + k_col + d] * expf(b_last[d] - b);
    }
  }
  for (int d = threadIdx.x; d < dim; d += blockDim.x)
    chunk_decay[((size_t)chunk * heads + head) * dim + d] = expf(b_last[d]);
  __syncthreads();
  // a warp owns kChunkRows state rows that follow each other, a lane the value columns lane, lane + 32, ...
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int i0 = warp * kChunkRows;
  const bool whole = dim % 4 == 0 && i0 + kChunkRows <= dim;
  float u[kChunkRows][kChunkCols] = {};
  for (int j = 0; j < n; ++j) {
    float vv[kChunkCols], kv[kChunkRows];
#pragma unroll
    for (int c = 0; c < kChunkCols; ++c) vv[c] = lane + 32 * c < vdim ? v_s[j * vdim + lane + 32 * c] : 0.f;
    if (whole) {
#pragma unroll
      for (int r = 0; r < kChunkRows; r += 4) {
        const float4 k4 = *reinterpret_cast<const float4*>(k_s + j * dim + i0 + r);
        kv[r] = k4.x; kv[r + 1] = k4.y; kv[r + 2] = k4.z; kv[r + 3] = k4.w;
      }
    } else {
#pragma unroll
      for (int r = 0; r < kChunkRows; ++r) kv[r] = i0 + r < dim ? k_s[j * dim + i0 + r] : 0.f;
    }
#pragma unroll
    for (int r = 0; r < kChunkRows; ++r)
#pragma unroll
      for (int c = 0; c < kChunkCols; ++c) u[r][c] = fmaf(kv[r], vv[c], u[r][c]);
  }
  float* dst = chunk_state + ((size_t)chunk * heads + head) * dim * vdim;
#pragma unroll
  for (int r = 0; r < kChunkRows; ++r) {
    const int i = i0 + r;
    if (i >= dim) continue;
#pragma unroll
    for (int c = 0; c < kChunkCols; ++c)
      if (lane + 32 * c < vdim) dst[(size_t)i * vdim + lane + 32 * c] = u[r][c];
  }
}

// (2) grid: (requests, heads, blocks over dim * vdim)
__global__ void gla_chunk_prefix_kernel(float* __restrict__ chunk_state, const float* __restrict__ chunk_decay,
                                        float* __restrict__ state, const int* __restrict__ request_chunk_start,
                                        const int* __restrict__ slots, const int* __restrict__ request_active,
                                        int heads, int dim, int vdim, int max_slots, int* err) {
  pdl_wait();
  pdl_trigger();
  const int request = blockIdx.x, head = blockIdx.y;
  const int e = blockIdx.z * blockDim.x + threadIdx.x;
  if (e >= dim * vdim) return;
  const int slot = slots[request];
  if (slot < 0 || slot >= max_slots) {
    if (e == 0) atomicOr(err, kErrBadRequest);
    return;
  }
  const int d = e / vdim;
  float* cell = state + ((size_t)slot * heads + head) * dim * vdim + e;
  float s = *cell;
  const size_t stride = (size_t)heads * dim * vdim, decay_stride = (size_t)heads * dim;
  const int last = request_chunk_start[request + 1];
  // eight chunks at a time: their sums are asked for together, before the first store, so that the walk waits
  // for memory once per eight chunks and not once per chunk
  constexpr int kBatch = 8;
  for (int chunk = request_chunk_start[request]; chunk < last; chunk += kBatch) {
    float* u = chunk_state + ((size_t)chunk * heads + head) * dim * vdim + e;
    const float* b = chunk_decay + ((size_t)chunk * heads + head) * dim + d;
    float gained[kBatch], power[kBatch];
#pragma unroll
    for (int x = 0; x < kBatch; ++x) {
      const bool in = chunk + x < last;
      gained[x] = in ? u[x * stride] : 0.f;
      power[x] = in ? b[x * decay_stride] : 1.f;
    }
#pragma unroll
    for (int x = 0; x < kBatch; ++x) {
      if (chunk + x < last) {
        u[x * stride] = s;
        s = fmaf(power[x], s, gained[x]);
      }
    }
  }
  if (request_active[request]) *cell = s;
}

// (3) outputs of a chunk from the state before it and the chunk's own tokens
__global__ void __launch_bounds__(kScanWarps * 32)
gla_chunk_output_kernel(GlaRows in, float* __restrict__ out, int out_stride, const float* __restrict__ chunk_state,
                        const int* __restrict__ chunk_row, const int* __restrict__ chunk_count, int heads, int dim,
                        int vdim) {
  extern __shared__ __align__(16) float smem[];
  const int ld = dim + 1;                         // rows that lanes walk side by side are padded by one element
  float* q_s = smem;                              // [kChunk][dim]
  float* v_s = q_s + kChunk * dim;                // [kChunk][vdim]
  float* k_s = v_s + kChunk * vdim;               // [kChunk][dim + 1]
  float* b_s = k_s + kChunk * ld;                 // [kChunk][dim + 1]
  float* a_s = b_s + kChunk * ld;                 // [kChunk][kChunk]
  pdl_wait();
  pdl_trigger();
  const int chunk = blockIdx.x, head = blockIdx.y;
  const int row0 = chunk_row[chunk], n = chunk_count[chunk];
  stage_rows(q_s, dim, in.proj, in.proj_stride, row0, n, in.q_off + head * dim, dim, in.q_scale);
  stage_rows(k_s, ld, in.proj, in.proj_stride, row0, n, in.k_off + head * dim, dim, 1.f);
  stage_rows(v_s, vdim, in.proj, in.proj_stride, row0, n, in.v_off + head * vdim, vdim, 1.f);
  // the sums in units of log 2: every exponential below is one exp2
  stage_rows(b_s, ld, in.z, in.z_stride, row0, n, head * dim, dim, 1.4426950408889634f);
  __syncthreads();
  // a[i][j] = sum_d q_i[d] k_j[d] exp(b_i[d] - b_j[d]) for j <= i.  Only those pairs are dealt out: pair p is
  // (i, j) with p = i (i + 1) / 2 + j, so neighbouring lanes mostly share i and walk neighbouring rows j
  const int pairs = n * (n + 1) / 2;
  for (int p = threadIdx.x; p < pairs; p += blockDim.x) {
    int i = (int)((sqrtf(8.f * (float)p + 1.f) - 1.f) * 0.5f);
    while (i * (i + 1) / 2 > p) --i;
    while ((i + 1) * (i + 2) / 2 <= p) ++i;
    const int j = p - i * (i + 1) / 2;
    const float* qi = q_s + i * dim;
    const float* bi = b_s + i * ld;
    const float* kj = k_s + j * ld;
    const float* bj = b_s + j * ld;
    float dot = 0.f, dot2 = 0.f;       // two chains
    int x = 0;
    for (; x + 2 <= dim; x += 2) {
      dot = fmaf(qi[x] * kj[x], exp2f(bi[x] - bj[x]), dot);
      dot2 = fmaf(qi[x + 1] * kj[x + 1], exp2f(bi[x + 1] - bj[x + 1]), dot2);
    }
    if (x < dim) dot = fmaf(qi[x] * kj[x], exp2f(bi[x] - bj[x]), dot);
    a_s[i * kChunk + j] = dot + dot2;
  }
  __syncthreads();
  // what the carried state is read with: q_i * exp(b_i)
  for (int e = threadIdx.x; e < n * dim; e += blockDim.x) {
    const int i = e / dim, x = e % dim;
    q_s[e] *= exp2f(b_s[i * ld + x]);
  }
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const float* before = chunk_state + ((size_t)chunk * heads + head) * dim * vdim;
  // a warp takes tokens warp, warp + 8, ...; a lane the value columns lane, lane + 32, ...
  constexpr int kTokens = kChunk / kScanWarps;
  float acc[kTokens][kChunkCols] = {};
  const int dim4 = dim % 4 == 0 ? dim : 0;       // four state rows a step where the q rows allow 16-byte loads
  for (int x = 0; x < dim4; x += 4) {
    float sv[4][kChunkCols];
#pragma unroll
    for (int y = 0; y < 4; ++y)
#pragma unroll
      for (int c = 0; c < kChunkCols; ++c) sv[y][c] = lane + 32 * c < vdim ? before[(size_t)(x + y) * vdim + lane + 32 * c] : 0.f;
#pragma unroll
    for (int t = 0; t < kTokens; ++t) {
      const int i = warp + kScanWarps * t;
      const float4 q4 = i < n ? *reinterpret_cast<const float4*>(q_s + i * dim + x) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int c = 0; c < kChunkCols; ++c) {
        acc[t][c] = fmaf(q4.x, sv[0][c], acc[t][c]);
        acc[t][c] = fmaf(q4.y, sv[1][c], acc[t][c]);
        acc[t][c] = fmaf(q4.z, sv[2][c], acc[t][c]);
        acc[t][c] = fmaf(q4.w, sv[3][c], acc[t][c]);
      }
    }
  }
  for (int x = dim4; x < dim; ++x) {
    float sv[kChunkCols];
#pragma unroll
    for (int c = 0; c < kChunkCols; ++c) sv[c] = lane + 32 * c < vdim ? before[(size_t)x * vdim + lane + 32 * c] : 0.f;
#pragma unroll
    for (int t = 0; t < kTokens; ++t) {
      const int i = warp + kScanWarps * t;
      const float qv = i < n ? q_s[i * dim + x] : 0.f;
#pragma unroll
      for (int c = 0; c < kChunkCols; ++c) acc[t][c] = fmaf(qv, sv[c], acc[t][c]);
    }
  }
  for (int j = 0; j < n; ++j) {
    float vv[kChunkCols];
#pragma unroll
    for (int c = 0; c < kChunkCols; ++c) vv[c] = lane + 32 * c < vdim ? v_s[j * vdim + lane + 32 * c] : 0.f;
#pragma unroll
    for (int t = 0; t < kTokens; ++t) {
      const int i = warp + kScanWarps * t;
      const float av = (i < n && j <= i) ? a_s[i * kChunk + j] : 0.f;
#pragma unroll
      for (int c = 0; c < kChunkCols; ++c) acc[t][c] = fmaf(av, vv[c], acc[t][c]);
    }
  }
#pragma unroll
  for (int t = 0; t < kTokens; ++t) {
    const int i = warp + kScanWarps * t;
    if (i >= n) continue;
#pragma unroll
    for (int c = 0; c < kChunkCols; ++c)
      if (lane + 32 * c < vdim) out[(size_t)(row0 + i) * out_stride + head * vdim + lane + 32 * c] = acc[t][c];
  }
}

}  // namespace cie

using namespace cie;

static int check_rows(const char* name, const GlaRows& in, int heads, int dim, int vdim) {
  if (heads < 1 || dim < 1 || vdim < 1) CIE_FAIL("%s: %d heads of key size %d and value size %d", name, heads, dim, vdim);
  if (!(in.inv_tau > 0.f)) CIE_FAIL("%s: the decay's temperature must be positive", name);
  if (!in.proj || !in.z || !in.z_bias) CIE_FAIL("%s: q/k/v rows, decay logits and their bias are all needed", name);
  return 0;
}

extern "C" int cie_gla_scan_max_dim() { return kScanWarps * kScanRows; }
extern "C" int cie_gla_chunk_tokens() { return kChunk; }
extern "C" int cie_gla_chunk_max_dim() { return kChunkDim; }

// proj: float32 [tokens][proj_stride] with q, k, v at columns q_off, k_off, v_off (heads side by side); z: float32
// [tokens][z_stride] decay logits (heads x dim) still without z_bias [heads * dim]; out: float32
// [tokens][out_stride], head h at column h * vdim; state: float32 [max_slots][heads][dim][vdim].
extern "C" int cie_gla_scan(const float* proj, int proj_stride, int q_off, int k_off, int v_off, const float* z,
                            int z_stride, const float* z_bias, float inv_tau, float q_scale, float* out,
                            int out_stride, float* state, const int* query_start, const int* slots,
                            const int* request_active, int requests, int heads, int dim, int vdim, int max_slots,
                            int* err, void* stream) {
  if (requests <= 0) return 0;
  const GlaRows in{proj, proj_stride, q_off, k_off, v_off, z, z_stride, z_bias, inv_tau, q_scale};
  if (check_rows("gla_scan", in, heads, dim, vdim)) return 1;
  if (dim > kScanWarps * kScanRows) CIE_FAIL("gla_scan: key size %d is above %d", dim, kScanWarps * kScanRows);
  dim3 grid(requests, heads, (vdim + kScanColumns - 1) / kScanColumns);
  CIE_LAUNCH("gla_scan", gla_scan_kernel, grid, dim3(kScanWarps * 32), 0, (cudaStream_t)stream, in, out, out_stride,
             state, query_start, slots, request_active, heads, dim, vdim, max_slots, err);
  return 0;
}

// The chunked form.  chunk_state: float32 scratch [chunks][heads][dim][vdim]; chunk_decay: [chunks][heads][dim].
// z is overwritten (with the running sums of the decays' logarithms inside every chunk).
extern "C" int cie_gla_chunked(const float* proj, int proj_stride, int q_off, int k_off, int v_off, float* z,
                               int z_stride, const float* z_bias, float inv_tau, float q_scale, float* out,
                               int out_stride, float* state, float* chunk_state, float* chunk_decay,
                               const int* chunk_row, const int* chunk_count, const int* request_chunk_start,
                               const int* slots, const int* request_active, int chunks, int requests, int heads,
                               int dim, int vdim, int max_slots, int* err, void* stream) {
  if (chunks <= 0 || requests <= 0) return 0;
  const GlaRows in{proj, proj_stride, q_off, k_off, v_off, z, z_stride, z_bias, inv_tau, q_scale};
  if (check_rows("gla_chunked", in, heads, dim, vdim)) return 1;
  if (dim > kChunkDim || vdim > kChunkDim)
    CIE_FAIL("gla_chunked: key / value sizes %d / %d are above %d", dim, vdim, kChunkDim);
  cudaStream_t s = (cudaStream_t)stream;
  const size_t smem1 = (size_t)kChunk * (dim + vdim) * sizeof(float);
  const size_t smem3 = (size_t)kChunk * (dim + vdim + 2 * (dim + 1) + kChunk) * sizeof(float);
  static bool raised = false;
  if (!raised) {
    if (cudaFuncSetAttribute(gla_chunk_state_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024) != cudaSuccess ||
        cudaFuncSetAttribute(gla_chunk_output_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024) != cudaSuccess)
      CIE_FAIL("gla_chunked: cannot raise the shared memory limit");
    raised = true;
  }
  dim3 grid(chunks, heads), block(kScanWarps * 32);
  dim3 grid2(requests, heads, (dim * vdim + 255) / 256);
  int sum_threads = 32;
  while (sum_threads < dim) sum_threads <<= 1;
  CIE_LAUNCH("gla_decay_sums", gla_decay_sums_kernel, grid, dim3(sum_threads), 0, s, z, z_stride, z_bias, inv_tau,
             chunk_row, chunk_count, dim);
  CIE_LAUNCH("gla_chunk_state", gla_chunk_state_kernel, grid, block, smem1, s, in, chunk_state, chunk_decay, chunk_row,
             chunk_count, heads, dim, vdim);
  CIE_LAUNCH("gla_chunk_prefix", gla_chunk_prefix_kernel, grid2, dim3(256), 0, s, chunk_state,
             (const float*)chunk_decay, state, request_chunk_start, slots, request_active, heads, dim, vdim,
             max_slots, err);
  CIE_LAUNCH("gla_chunk_output", gla_chunk_output_kernel, grid, block, smem3, s, in, out, out_stride,
             (const float*)chunk_state, chunk_row, chunk_count, heads, dim, vdim);
  return 0;
}
