// Causal attention of a ragged batch over the paged cache, one warp per (token, query head).
// Any head size up to 256, any page size, any number of heads and groups, float32 or bfloat16
// storage; all arithmetic is float32.  This is the 32-bit path's attention and the fallback for
// head or page sizes the tensor-core kernels do not take.
//
// Formula (zeeshan8281/cloud-inference-from-scratch src/cloud_engine/kernel.py:356-405): for query
// token t at position p of its request, keys 0..p (or p-window+1..p), s = (q.k) * scale,
// running-maximum softmax, out = sum(p v) / sum(p); query head h reads kv head h / (Hq/Hkv).
// Keys are visited in blocks of 32 counted from the first visible key, so the result for a
// token depends only on its request's keys, not on the batch, the cut or the pages used.
//
// Two generalisations: value heads of a size of their own (`vdim`), and
// a logarithmic distance penalty per query head, s = (q.k) * scale - r1[h] * log(1 + r2[h] * (p - j))
// for a key at position j (r1 == nullptr: none).
//
// `keep_first` > 0 (with a window): the first keep_first keys of the request stay visible after the
// window has moved past them; the visible keys are then 0..keep_first-1 and p-window+1..p, visited in
// that order as one list.
//
// `sinks` != nullptr: the softmax denominator of query head h holds one more term exp(sinks[h]), which has no
// key and no value and is not scaled.
#include "common.cuh"

#include <cfloat>

CIE_DEFINE_LAST_ERROR()

namespace cie {

constexpr int kMaxDim = 256;
constexpr int kWarps = 4;

template <typename T>
__global__ void __launch_bounds__(kWarps * 32)
attention_generic_kernel(const T* __restrict__ q, int q_stride, T* __restrict__ out, int out_stride,
                         const T* __restrict__ k_pool, const T* __restrict__ v_pool,
                         const int* __restrict__ positions, const int* __restrict__ request_of_token,
                         const int* __restrict__ table, int table_width, int num_pages, int tokens,
                         int q_heads, int kv_heads, int dim, int vdim, int page_size, float scale, int window,
                         int keep_first, const float* __restrict__ r1, const float* __restrict__ r2,
                         const float* __restrict__ sinks, int* err) {
  __shared__ float q_s[kWarps][kMaxDim];
  __shared__ float p_s[kWarps][32];
  __shared__ long long off_s[kWarps][32];
  pdl_wait();
  pdl_trigger();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int item = blockIdx.x * kWarps + warp;
  if (item >= tokens * q_heads) return;
  const int t = item / q_heads, h = item % q_heads;
  const int kvh = h / (q_heads / kv_heads);
  const int pos = positions[t];
  const int request = request_of_token[t];
  const int* row = table + (size_t)request * table_width;
  const int length = pos + 1;
  int first = (window > 0 && length > window) ? length - window : 0;
  int kept = 0;                       // keys before the window that stay visible
  if (first > keep_first) kept = keep_first;
  else first = 0;
  const int visible = kept + length - first;
  const float penalty = r1 ? r1[h] : 0.f, reach = r1 ? r2[h] : 0.f;

  const T* qv = q + (size_t)t * q_stride + (size_t)h * dim;
  for (int d = lane; d < dim; d += 32) q_s[warp][d] = to_float(qv[d]);
  __syncwarp();

  float m = -FLT_MAX, l = 0.f;
  float acc[kMaxDim / 32];
#pragma unroll
  for (int i = 0; i < kMaxDim / 32; ++i) acc[i] = 0.f;

  for (int base = 0; base < visible; base += 32) {
    const int seen = base + lane;
    const bool valid = seen < visible;
    const int key = seen < kept ? seen : first + (seen - kept);
    long long offset = -1;
    if (valid) {
      const int index = key / page_size;
      const int page = index < table_width ? row[index] : -1;
      if (page < 0 || page >= num_pages) {
        atomicOr(err, kErrBadPage);
      } else {
        offset = ((long long)page * kv_heads + kvh) * page_size + key % page_size;   // slot; times dim or vdim
      }
    }
    float s = -FLT_MAX;
    if (offset >= 0) {
      const T* kr = k_pool + offset * dim;
      float dot = 0.f;
      for (int d = 0; d < dim; ++d) dot = fmaf(q_s[warp][d], to_float(kr[d]), dot);
      s = dot * scale;
      if (r1) s -= penalty * log1pf(reach * (float)(pos - key));
    }
    const float m_new = fmaxf(m, warp_max(s));
    const float p = offset >= 0 ? expf(s - m_new) : 0.f;
    const float alpha = expf(m - m_new);
    l = l * alpha + warp_sum(p);
    m = m_new;
    p_s[warp][lane] = p;
    off_s[warp][lane] = offset;
    __syncwarp();
#pragma unroll
    for (int i = 0; i < kMaxDim / 32; ++i) acc[i] *= alpha;
    const int count = min(32, visible - base);
    for (int j = 0; j < count; ++j) {
      const long long o = off_s[warp][j];
      if (o < 0) continue;
      const float pj = p_s[warp][j];
      const T* vr = v_pool + o * vdim;
#pragma unroll
      for (int i = 0; i < kMaxDim / 32; ++i) {
        const int d = lane + 32 * i;
        if (d < vdim) acc[i] = fmaf(pj, to_float(vr[d]), acc[i]);
      }
    }
    __syncwarp();
  }
  T* o = out + (size_t)t * out_stride + (size_t)h * vdim;
  float keep = 1.f;
  if (sinks) {      // the sink joins the denominator, measured from the larger of the two maxima
    const float top = fmaxf(m, sinks[h]);
    keep = expf(m - top);
    l = l * keep + expf(sinks[h] - top);
  }
  const float inv = l > 0.f ? keep / l : 0.f;
#pragma unroll
  for (int i = 0; i < kMaxDim / 32; ++i) {
    const int d = lane + 32 * i;
    if (d < vdim) o[d] = from_float<T>(acc[i] * inv);
  }
}

// ---------------------------------------------------------------- the heads of a group together
// One CTA per (token, kv head, up to 8 query heads of its group): the heads share every key and value
// row that is read.  Eight warps take blocks of 32 keys in turn; inside a block a lane owns one key
// and reads its whole row with 16-byte loads (scores of all heads against it), then owns value
// columns (lane, lane + 32, ...) while the block's keys go by.  Every warp keeps a running maximum,
// sum and output of its own; they are joined in warp order at the end.  Same formula and options as
// above; key sizes a multiple of the 16-byte vector up to 256, value sizes up to 128.
constexpr int kGroupHeads = 8, kGroupWarps = 8, kGroupMaxV = 128;

template <typename T> struct Vec16;
template <> struct Vec16<float> { static constexpr int n = 4; };
template <> struct Vec16<__nv_bfloat16> { static constexpr int n = 8; };

__device__ __forceinline__ void stage16(void* dst, const void* src) {
  const unsigned d = (unsigned)__cvta_generic_to_shared(dst);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(src) : "memory");
}
__device__ __forceinline__ void stage_wait() {
  asm volatile("cp.async.commit_group;" ::: "memory");
  asm volatile("cp.async.wait_group 0;" ::: "memory");
}

// kStaged: a warp first brings the key and value rows of its 32 keys into shared memory with
// asynchronous 16-byte copies, all in flight at once (one trip to memory a block instead of one per
// row piece), and reads them from there; rows of 16-bit elements whose sizes are multiples of 8.
template <typename T, bool kStaged>
__global__ void __launch_bounds__(kGroupWarps * 32)
attention_group_kernel(const T* __restrict__ q, int q_stride, T* __restrict__ out, int out_stride,
                       const T* __restrict__ k_pool, const T* __restrict__ v_pool,
                       const int* __restrict__ positions, const int* __restrict__ request_of_token,
                       const int* __restrict__ table, int table_width, int num_pages, int q_heads,
                       int kv_heads, int dim, int vdim, int page_size, float scale, int window, int keep_first,
                       const float* __restrict__ r1, const float* __restrict__ r2,
                       const float* __restrict__ sinks, int splits,
                       float* __restrict__ shares, int* __restrict__ tickets, int* err) {
  // splits > 1: the keys of a token are cut into that many ranges, one CTA each (blockIdx.x = token *
  // splits + range); a CTA leaves its maximum, sum and unnormalised output in `shares`, and whoever
  // draws the unit's last ticket joins them in range order (tickets are zero between launches)
  constexpr int V = Vec16<T>::n;
  extern __shared__ __align__(16) float group_smem[];
  float* q_s = group_smem;                                   // [kGroupHeads][dim]
  float* p_s = q_s + kGroupHeads * dim;                      // [warps][kGroupHeads][32]
  float* o_s = p_s + kGroupWarps * kGroupHeads * 32;         // [warps][kGroupHeads][kGroupMaxV]
  float* ml_s = o_s + kGroupWarps * kGroupHeads * kGroupMaxV;  // [warps][kGroupHeads][2]
  long long* slot_s = reinterpret_cast<long long*>(ml_s + kGroupWarps * kGroupHeads * 2);   // [warps][32]
  const int k_ld = dim + 16 / (int)sizeof(T);          // staged key rows are padded by 16 bytes: no bank conflicts
  T* k_stage = reinterpret_cast<T*>(slot_s + kGroupWarps * 32);                 // [warps][32][k_ld]
  T* v_stage = k_stage + (size_t)kGroupWarps * 32 * k_ld;                      // [warps][32][vdim]
  pdl_wait();
  pdl_trigger();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x / splits, split = blockIdx.x % splits, kvh = blockIdx.y;
  const int group = q_heads / kv_heads;
  const int h0 = blockIdx.z * kGroupHeads, heads = min(kGroupHeads, group - h0);
  const int pos = positions[t];
  const int* row = table + (size_t)request_of_token[t] * table_width;
  const int length = pos + 1;
  int first = (window > 0 && length > window) ? length - window : 0;
  int kept = 0;                       // keys before the window that stay visible
  if (first > keep_first) kept = keep_first;
  else first = 0;
  const int visible = kept + length - first;
  // this CTA's keys: whole blocks of 32 of the list of visible keys
  const int per = ((visible + splits - 1) / splits + 31) / 32 * 32;
  const int my_first = split * per, my_end = min(visible, my_first + per);
  for (int e = threadIdx.x; e < kGroupHeads * dim; e += blockDim.x) {
    const int h = e / dim, d = e % dim;
    q_s[e] = h < heads ? to_float(q[(size_t)t * q_stride + (size_t)(kvh * group + h0 + h) * dim + d]) : 0.f;
  }
  float penalty[kGroupHeads], reach[kGroupHeads];
#pragma unroll
  for (int h = 0; h < kGroupHeads; ++h) {
    penalty[h] = (r1 && h < heads) ? r1[kvh * group + h0 + h] : 0.f;
    reach[h] = (r1 && h < heads) ? r2[kvh * group + h0 + h] : 0.f;
  }
  __syncthreads();
  float m[kGroupHeads], l[kGroupHeads], acc[kGroupHeads][kGroupMaxV / 32];
#pragma unroll
  for (int h = 0; h < kGroupHeads; ++h) {
    m[h] = -FLT_MAX;
    l[h] = 0.f;
#pragma unroll
    for (int c = 0; c < kGroupMaxV / 32; ++c) acc[h][c] = 0.f;
  }
  float* my_p = p_s + warp * kGroupHeads * 32;
  long long* my_slot = slot_s + warp * 32;
  for (int base = my_first + warp * 32; base < my_end; base += kGroupWarps * 32) {
    const int seen = base + lane;
    const int key = seen < kept ? seen : first + (seen - kept);
    long long slot = -1;
    if (seen < my_end) {
      const int index = key / page_size;
      const int page = index < table_width ? row[index] : -1;
      if (page < 0 || page >= num_pages) atomicOr(err, kErrBadPage);
      else slot = ((long long)page * kv_heads + kvh) * page_size + key % page_size;
    }
    float dot[kGroupHeads];
#pragma unroll
    for (int h = 0; h < kGroupHeads; ++h) dot[h] = 0.f;
    T* my_k = k_stage + ((size_t)warp * 32 + lane) * k_ld;
    T* my_v = v_stage + (size_t)warp * 32 * vdim;
    if constexpr (kStaged) {
      if (slot >= 0) {
        for (int d0 = 0; d0 < dim; d0 += V) stage16(my_k + d0, k_pool + slot * dim + d0);
        for (int d0 = 0; d0 < vdim; d0 += V) stage16(my_v + (size_t)lane * vdim + d0, v_pool + slot * vdim + d0);
      }
      stage_wait();
      __syncwarp();
    }
    if (slot >= 0) {
      const T* kr = kStaged ? my_k : k_pool + slot * dim;
      for (int d0 = 0; d0 < dim; d0 += V) {
        const uint4 raw = *reinterpret_cast<const uint4*>(kr + d0);
        const T* kv = reinterpret_cast<const T*>(&raw);
#pragma unroll
        for (int x = 0; x < V; ++x) {
          const float kf = to_float(kv[x]);
#pragma unroll
          for (int h = 0; h < kGroupHeads; ++h) dot[h] = fmaf(q_s[h * dim + d0 + x], kf, dot[h]);
        }
      }
    }
    const float distance = (float)(pos - key);
#pragma unroll
    for (int h = 0; h < kGroupHeads; ++h) {
      float s = -FLT_MAX;
      if (slot >= 0) {
        s = dot[h] * scale;
        if (r1) s -= penalty[h] * log1pf(reach[h] * distance);
      }
      const float m_new = fmaxf(m[h], warp_max(s));
      const float p = slot >= 0 ? expf(s - m_new) : 0.f;
      const float alpha = expf(m[h] - m_new);
      l[h] = l[h] * alpha + warp_sum(p);
      m[h] = m_new;
      my_p[h * 32 + lane] = p;
#pragma unroll
      for (int c = 0; c < kGroupMaxV / 32; ++c) acc[h][c] *= alpha;
    }
    my_slot[lane] = slot;
    __syncwarp();
    const int count = min(32, my_end - base);
    for (int j = 0; j < count; ++j) {
      const long long o = my_slot[j];
      if (o < 0) continue;
      const T* vr = kStaged ? my_v + (size_t)j * vdim : v_pool + o * vdim;
      float vv[kGroupMaxV / 32];
#pragma unroll
      for (int c = 0; c < kGroupMaxV / 32; ++c) vv[c] = lane + 32 * c < vdim ? to_float(vr[lane + 32 * c]) : 0.f;
#pragma unroll
      for (int h = 0; h < kGroupHeads; ++h) {
        const float pj = my_p[h * 32 + j];
#pragma unroll
        for (int c = 0; c < kGroupMaxV / 32; ++c) acc[h][c] = fmaf(pj, vv[c], acc[h][c]);
      }
    }
    __syncwarp();
  }
  // ---- join the warps, in warp order
#pragma unroll
  for (int h = 0; h < kGroupHeads; ++h) {
#pragma unroll
    for (int c = 0; c < kGroupMaxV / 32; ++c) o_s[(warp * kGroupHeads + h) * kGroupMaxV + lane + 32 * c] = acc[h][c];
    if (lane == 0) {
      ml_s[(warp * kGroupHeads + h) * 2] = m[h];
      ml_s[(warp * kGroupHeads + h) * 2 + 1] = l[h];
    }
  }
  __syncthreads();
  const size_t unit = ((size_t)t * kv_heads + kvh) * gridDim.z + blockIdx.z;
  constexpr int kShare = kGroupMaxV + 2;      // floats of one head's share: output, then maximum and sum
  float* my_share = shares ? shares + (unit * splits + split) * kGroupHeads * kShare : nullptr;
  for (int e = threadIdx.x; e < heads * vdim; e += blockDim.x) {
    const int h = e / vdim, d = e % vdim;
    const bool sunk = sinks != nullptr && splits == 1;     // with key ranges the sink joins when they are joined
    const float sink = sunk ? sinks[kvh * group + h0 + h] : -FLT_MAX;
    float top = sink;
#pragma unroll
    for (int w = 0; w < kGroupWarps; ++w) top = fmaxf(top, ml_s[(w * kGroupHeads + h) * 2]);
    float sum = sunk ? expf(sink - top) : 0.f, value = 0.f;
#pragma unroll
    for (int w = 0; w < kGroupWarps; ++w) {
      const float share = expf(ml_s[(w * kGroupHeads + h) * 2] - top);
      sum = fmaf(share, ml_s[(w * kGroupHeads + h) * 2 + 1], sum);
      value = fmaf(share, o_s[(w * kGroupHeads + h) * kGroupMaxV + d], value);
    }
    if (splits == 1) {
      out[(size_t)t * out_stride + (size_t)(kvh * group + h0 + h) * vdim + d] = from_float<T>(sum > 0.f ? value / sum : 0.f);
    } else {
      my_share[h * kShare + d] = value;
      if (d == 0) {
        my_share[h * kShare + kGroupMaxV] = top;
        my_share[h * kShare + kGroupMaxV + 1] = sum;
      }
    }
  }
  if (splits == 1) return;
  __shared__ int last_s;
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const int ticket = atomicAdd(tickets + unit, 1);
    last_s = ticket == splits - 1;
    if (last_s) tickets[unit] = 0;
  }
  __syncthreads();
  if (!last_s) return;
  __threadfence();
  const float* unit_shares = shares + unit * splits * kGroupHeads * kShare;
  for (int e = threadIdx.x; e < heads * vdim; e += blockDim.x) {
    const int h = e / vdim, d = e % vdim;
    const float sink = sinks ? sinks[kvh * group + h0 + h] : -FLT_MAX;
    float top = sink;
    for (int r = 0; r < splits; ++r) top = fmaxf(top, __ldcg(unit_shares + (r * kGroupHeads + h) * kShare + kGroupMaxV));
    float sum = sinks ? expf(sink - top) : 0.f, value = 0.f;
    for (int r = 0; r < splits; ++r) {
      const float* part = unit_shares + (r * kGroupHeads + h) * kShare;
      const float share = expf(__ldcg(part + kGroupMaxV) - top);
      sum = fmaf(share, __ldcg(part + kGroupMaxV + 1), sum);
      value = fmaf(share, __ldcg(part + d), value);
    }
    out[(size_t)t * out_stride + (size_t)(kvh * group + h0 + h) * vdim + d] = from_float<T>(sum > 0.f ? value / sum : 0.f);
  }
}

}  // namespace cie

using namespace cie;

extern "C" int cie_attention_group_share_floats() { return kGroupHeads * (kGroupMaxV + 2); }

// q: rows of q_stride elements, query head h of token t at q[t*q_stride + h*dim].
// out: [tokens, out_stride], head h at column h*vdim.  Pools: [pages][kv_heads][page_size][dim or vdim].
// splits > 1 (the kernel that shares keys among a group's heads only; ignored otherwise): a token's
// keys are cut into that many ranges with a CTA each; `shares` holds tokens * kv_heads *
// ceil(group / 8) * splits * cie_attention_group_share_floats() floats and `tickets` one int, zero, per
// (token, kv head, 8 heads).
// sinks: float32 [q_heads] or nullptr.
extern "C" int cie_attention_generic_sink(const void* q, int q_stride, void* out, int out_stride,
                                          const void* k_pool, const void* v_pool, const int* positions,
                                          const int* request_of_token, const int* table, int table_width,
                                          int num_pages, int tokens, int q_heads, int kv_heads, int dim,
                                          int vdim, int page_size, float scale, int window,
                                          const float* r1, const float* r2, int splits, float* shares,
                                          int* tickets, int keep_first, const float* sinks, int dtype, int* err,
                                          void* stream) {
  if (tokens <= 0) return 0;
  if (keep_first < 0) CIE_FAIL("attention_generic: %d kept keys", keep_first);
  if (splits < 1 || (splits > 1 && (!shares || !tickets))) CIE_FAIL("attention_generic: %d key ranges need shares and tickets", splits);
  if (dim > kMaxDim || dim < 1 || vdim > kMaxDim || vdim < 1)
    CIE_FAIL("attention_generic: head sizes %d / %d are outside 1..%d", dim, vdim, kMaxDim);
  if (kv_heads < 1 || q_heads % kv_heads) CIE_FAIL("attention_generic: %d query heads do not divide over %d kv heads", q_heads, kv_heads);
  if (page_size < 1) CIE_FAIL("attention_generic: page size %d", page_size);
  if ((r1 == nullptr) != (r2 == nullptr)) CIE_FAIL("attention_generic: the distance penalty needs both of its vectors");
  const long long items = (long long)tokens * q_heads;
  const int blocks = (int)((items + kWarps - 1) / kWarps);
  cudaStream_t s = (cudaStream_t)stream;
  // the kernel that shares the keys among the heads of a group, where the sizes allow its 16-byte loads
  const int vec = dtype == kFloat32 ? 4 : 8;
  static const bool grouped = [] { const char* v = getenv("CIE_ATTENTION_GROUPED"); return !(v && v[0] == '0'); }();
  if (grouped && dim % vec == 0 && vdim <= kGroupMaxV && (dtype == kFloat32 || dtype == kBFloat16) &&
      (reinterpret_cast<uintptr_t>(k_pool) & 15) == 0) {
    const int group = q_heads / kv_heads;
    const size_t base = sizeof(float) * ((size_t)kGroupHeads * dim + kGroupWarps * kGroupHeads * (32 + kGroupMaxV + 2)) +
                        sizeof(long long) * kGroupWarps * 32;
    // bfloat16 rows are staged in shared memory where value rows, too, are whole 16-byte pieces
    const bool staged = dtype == kBFloat16 && vdim % 8 == 0 && (reinterpret_cast<uintptr_t>(v_pool) & 15) == 0;
    const size_t smem = base + (staged ? (size_t)kGroupWarps * 32 * (dim + 8 + vdim) * sizeof(__nv_bfloat16) : 0);
    dim3 grid(tokens * splits, kv_heads, (group + kGroupHeads - 1) / kGroupHeads);
#define CIE_GROUP(T, S)                                                                                            \
  do {                                                                                                             \
    if (cudaFuncSetAttribute(attention_group_kernel<T, S>, cudaFuncAttributeMaxDynamicSharedMemorySize,            \
                             (int)smem) != cudaSuccess)                                                            \
      CIE_FAIL("attention_generic: cannot reserve %zu bytes of shared memory", smem);                              \
    CIE_LAUNCH("attention_group", (attention_group_kernel<T, S>), grid, dim3(kGroupWarps * 32), smem, s,            \
               (const T*)q, q_stride, (T*)out, out_stride, (const T*)k_pool, (const T*)v_pool, positions,          \
               request_of_token, table, table_width, num_pages, q_heads, kv_heads, dim, vdim, page_size, scale,    \
               window, keep_first, r1, r2, sinks, splits, shares, tickets, err);                                   \
  } while (0)
    if (dtype == kFloat32) CIE_GROUP(float, false);
    else if (staged) CIE_GROUP(__nv_bfloat16, true);
    else CIE_GROUP(__nv_bfloat16, false);
#undef CIE_GROUP
    return 0;
  }
  if (dtype == kFloat32) {
    CIE_LAUNCH("attention_generic", attention_generic_kernel<float>, dim3(blocks), dim3(kWarps * 32), 0, s,
        (const float*)q, q_stride, (float*)out, out_stride, (const float*)k_pool, (const float*)v_pool,
        positions, request_of_token, table, table_width, num_pages, tokens, q_heads, kv_heads, dim, vdim,
        page_size, scale, window, keep_first, r1, r2, sinks, err);
  } else if (dtype == kBFloat16) {
    CIE_LAUNCH("attention_generic", attention_generic_kernel<__nv_bfloat16>, dim3(blocks), dim3(kWarps * 32), 0, s,
        (const __nv_bfloat16*)q, q_stride, (__nv_bfloat16*)out, out_stride, (const __nv_bfloat16*)k_pool,
        (const __nv_bfloat16*)v_pool, positions, request_of_token, table, table_width, num_pages, tokens,
        q_heads, kv_heads, dim, vdim, page_size, scale, window, keep_first, r1, r2, sinks, err);
  } else {
    CIE_FAIL("attention_generic: unknown element type code %d", dtype);
  }
  return 0;
}
