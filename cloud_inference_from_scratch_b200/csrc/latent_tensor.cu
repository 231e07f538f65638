// Attention over cached latent rows on the tensor cores (bfloat16 pages; see latent.cu for the
// arithmetic and the plain kernel that serves every other case).
//
// One CTA per (token, group of 16 heads, key range): the 16 heads of a token are the 16 rows of an
// mma.sync tile, since all heads of a token read the same rows [c_j | kr_j].  In prompt portions a CTA
// takes two consecutive tokens (two row tiles), so that every key fragment it loads serves both.  Keys come 64 at a time
// into shared memory with cp.async (two buffers: tile i+1 is on its way while tile i is used) and
// serve twice, as the key operand of the scores and, their first `rank` columns, as the value
// operand of the sums.  Eight warps: for the scores warp w takes keys 8w .. 8w+7 of the tile over
// all of [rank + rot]; for the sums warp w takes latent columns w * CW .. (w + 1) * CW - 1 over all 64
// keys.  Between the two the softmax weights pass through shared memory as TWO bfloat16 terms
// (the weight rounded, and what the rounding left), so that 16 bits of a float32 weight's mantissa
// reach the sum; maxima, sums and the denominators are float32, and the query is rounded to
// bfloat16 once, after its plain part was carried into the latent space in float32.
//
// ranges == 1: the normalised sum (with the sink term, if any, in the denominator) goes to `out`
// [T, heads, rank]; else the CTA leaves (maximum, sum, unnormalised latent sum) in `part`
// [T, heads, ranges, rank + 2] for latent_merge (latent.cu), as the plain kernel does.
#include "common.cuh"

#include <cfloat>

CIE_DEFINE_LAST_ERROR()

namespace cie {

using bf16 = __nv_bfloat16;
constexpr int kWarps = 8;
constexpr int kRows = 16;        // heads of a CTA
constexpr int kTile = 64;        // keys of a tile

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool valid) {
  const int bytes = valid ? 16 : 0;  // 0: the 16 bytes are filled with zeros, nothing is read
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(smem_u32(dst)), "l"(src), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void ldsm_x2(uint32_t& r0, uint32_t& r1, const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];\n" : "=r"(r0), "=r"(r1) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void ldsm_x2_trans(uint32_t& r0, uint32_t& r1, const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];\n" : "=r"(r0), "=r"(r1) : "r"(smem_u32(p)));
}
// the same loads by shared-memory address (the conversion from a pointer is done once, outside the loops)
__device__ __forceinline__ void ldsm_x4_at(uint32_t (&r)[4], uint32_t address) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(address));
}
__device__ __forceinline__ void ldsm_x2_at(uint32_t& r0, uint32_t& r1, uint32_t address) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];\n" : "=r"(r0), "=r"(r1) : "r"(address));
}
__device__ __forceinline__ void ldsm_x2_trans_at(uint32_t& r0, uint32_t& r1, uint32_t address) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];\n" : "=r"(r0), "=r"(r1) : "r"(address));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ float quad_max(float v) {
  v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 1));
  return fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 2));
}
__device__ __forceinline__ float quad_sum(float v) {
  v += __shfl_xor_sync(0xffffffffu, v, 1);
  return v + __shfl_xor_sync(0xffffffffu, v, 2);
}

struct Layout {
  int depth;      // rank + rot rounded up to 16: the K extent of the scores
  int ld;         // elements of a shared-memory row: covers depth and 8 * column_width, plus 8 (an odd number of 16-byte units)
  int rows;       // query rows of a CTA: 16 heads of one token, or of two consecutive tokens
  __host__ __device__ static Layout of(int rank, int rot, int column_width, int row_tiles) {
    Layout l;
    l.depth = (rank + rot + 15) / 16 * 16;
    const int widest = l.depth > kWarps * column_width ? l.depth : kWarps * column_width;
    l.ld = widest + 8;
    l.rows = kRows * row_tiles;
    return l;
  }
  __host__ __device__ size_t bytes() const {
    return ((size_t)(rows + 2 * kTile) * ld + 2 * rows * (kTile + 8)) * sizeof(bf16) +
           (size_t)(2 * kWarps * rows) * sizeof(float) + 2 * kTile * sizeof(long long);
  }
};

// NT: 8-column tiles of the latent a warp sums (column width CW = 8 * NT; 8 warps cover rank <= 64 * NT).
// RT: row tiles of a CTA.  RT == 2 (prompt portions, ranges == 1): CTA b takes tokens 2b and 2b + 1; if they
// belong to one request they share every key tile (the later token sees one key more), else the CTA
// runs them one after the other.
template <int NT, int RT>
__global__ void __launch_bounds__(kWarps * 32)
latent_attention_tensor_kernel(const float* __restrict__ q_abs, const float* __restrict__ q_raw, int q_raw_stride,
                               int q_raw_head, float* __restrict__ out, float* __restrict__ part,
                               const bf16* __restrict__ c_pool, const bf16* __restrict__ r_pool,
                               const int* __restrict__ positions, const int* __restrict__ request_of_token,
                               const int* __restrict__ table, int table_width, int num_pages,
                               const float* __restrict__ inv_freq, float magnitude, int interleaved, int rot_dims,
                               const float* __restrict__ sink, int tokens, int heads, int rank, int rot, int page_size,
                               float scale, int range_keys, int ranges, int window, int* err) {
  extern __shared__ __align__(16) unsigned char shared_raw[];
  constexpr int CW = 8 * NT;
  constexpr int ROWS = kRows * RT;
  constexpr int PLD = kTile + 8;
  const Layout lay = Layout::of(rank, rot, CW, RT);
  const int ld = lay.ld;
  bf16* qs = reinterpret_cast<bf16*>(shared_raw);                 // [ROWS][ld]
  bf16* ks = qs + ROWS * ld;                                       // [2][64][ld]
  bf16* ps = ks + 2 * kTile * ld;                                  // [2 terms][ROWS][64 + 8]
  float* wmax = reinterpret_cast<float*>(ps + 2 * ROWS * PLD);     // [8 warps][ROWS]
  float* wsum = wmax + kWarps * ROWS;                              // [8 warps][ROWS]
  long long* row_of = reinterpret_cast<long long*>(wsum + kWarps * ROWS);   // [2][64]

  pdl_wait();
  pdl_trigger();
  const int h0 = blockIdx.y * kRows;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, tg = lane & 3;
  const int D = rank + rot;
  const int first_token = blockIdx.x * RT;
  const bool second = RT == 2 && first_token + 1 < tokens;
  const bool together = second && request_of_token[first_token + 1] == request_of_token[first_token];
  const int passes = (second && !together) ? 2 : 1;

  // shared-memory addresses of this lane's fragment rows: query rows, the keys of this warp, the
  // weights, and the latent columns of this warp (each plus a tile's offset inside the loops)
  const uint32_t q_at = smem_u32(qs + (lane & 15) * ld + (lane >> 4) * 8);
  const uint32_t k_at = smem_u32(ks + (warp * 8 + (lane & 7)) * ld + ((lane >> 3) & 1) * 8);
  const uint32_t p_at = smem_u32(ps + (lane & 15) * PLD + (lane >> 4) * 8);
  const uint32_t v_at = smem_u32(ks + (lane & 15) * ld + warp * CW);

  for (int pass = 0; pass < passes; ++pass) {
    // the tokens of the row tiles (-1: the tile is idle) and the keys this pass walks
    int token[RT], position[RT];
    token[0] = first_token + pass;
    position[0] = positions[token[0]];
    if (RT == 2) {
      token[RT - 1] = together ? first_token + 1 : -1;
      position[RT - 1] = together ? positions[first_token + 1] : position[0];
    }
    const int length = position[RT - 1] + 1;
    // window > 0: a token sees its last `window` keys (itself included); the walk starts at the first key the
    // earlier token of the tile sees, and the later token does not weigh that one
    int lowest[RT];
#pragma unroll
    for (int tile = 0; tile < RT; ++tile) lowest[tile] = window > 0 ? max(0, position[tile] + 1 - window) : 0;
    const int begin = lowest[0] + blockIdx.z * range_keys;
    if (begin >= length) continue;
    const int end = min(length, begin + range_keys);
    const int* pages = table + (size_t)request_of_token[token[0]] * table_width;

    __syncthreads();      // a pass before this one is done with everything
    // what no copy writes starts as zero (padding must not hold NaN patterns): the query rows, the weights,
    // and the columns of every key row beyond [rank + rot]; rows past the last key are zero-filled by the copies
    {
      const int pad = ld - D;
      for (int e = tid; e < ROWS * ld; e += blockDim.x) qs[e] = __float2bfloat16_rn(0.f);
      for (int e = tid; e < 2 * kTile * pad; e += blockDim.x) ks[(e / pad) * ld + D + e % pad] = __float2bfloat16_rn(0.f);
      for (int e = tid; e < 2 * ROWS * PLD; e += blockDim.x) ps[e] = __float2bfloat16_rn(0.f);
    }
    __syncthreads();

    // the query rows: the latent part as it comes, the rotated part rotated here, both rounded once
#pragma unroll
    for (int tile = 0; tile < RT; ++tile) {
      const int t = token[tile];
      if (t < 0) continue;
      bf16* rows = qs + tile * kRows * ld;
      for (int e = tid; e < kRows * rank; e += blockDim.x) {
        const int r = e / rank, d = e % rank;
        if (h0 + r < heads) rows[r * ld + d] = __float2bfloat16_rn(q_abs[((size_t)t * heads + h0 + r) * rank + d]);
      }
      for (int e = tid; e < kRows * (rot_dims / 2); e += blockDim.x) {
        const int r = e / (rot_dims / 2), i = e % (rot_dims / 2);
        if (h0 + r >= heads) continue;
        const float* qr = q_raw + (size_t)t * q_raw_stride + (size_t)(h0 + r) * q_raw_head;
        const int a = interleaved ? 2 * i : i, b = interleaved ? 2 * i + 1 : i + rot_dims / 2;
        float sn, cs;
        sincosf((float)position[tile] * inv_freq[i], &sn, &cs);
        sn *= magnitude;
        cs *= magnitude;
        const float u = qr[a], v = qr[b];
        rows[r * ld + rank + a] = __float2bfloat16_rn(u * cs - v * sn);
        rows[r * ld + rank + b] = __float2bfloat16_rn(v * cs + u * sn);
      }
      for (int e = tid; e < kRows * (rot - rot_dims); e += blockDim.x) {
        const int r = e / (rot - rot_dims), i = rot_dims + e % (rot - rot_dims);
        if (h0 + r < heads)
          rows[r * ld + rank + i] = __float2bfloat16_rn(q_raw[(size_t)t * q_raw_stride + (size_t)(h0 + r) * q_raw_head + i]);
      }
    }

    auto fetch = [&](int base, int buf) {
      // which row of the pools every key of the tile lives in
      if (tid < kTile) {
        long long r = -1;
        const int key = base + tid;
        if (key < end) {
          const int page = pages[key / page_size];
          if (page < 0 || page >= num_pages) atomicOr(err, kErrBadPage);
          else r = (long long)page * page_size + key % page_size;
        }
        row_of[buf * kTile + tid] = r;
      }
    };
    auto copy = [&](int buf) {
      // warp w brings keys 8w .. 8w + 7 of the tile, a lane every 32nd 16-byte piece of a row
      bf16* dst = ks + (size_t)buf * kTile * ld;
#pragma unroll
      for (int jj = 0; jj < kTile / kWarps; ++jj) {
        const int j = warp * (kTile / kWarps) + jj;
        const long long r = row_of[buf * kTile + j];
        const bool valid = r >= 0;
        const bf16* c_src = c_pool + (valid ? (size_t)r * rank : 0);
        const bf16* r_src = r_pool + (valid ? (size_t)r * rot : 0);
        bf16* row = dst + j * ld;
        for (int c = lane * 8; c < D; c += 256) {
          const bf16* src = c < rank ? c_src + (valid ? c : 0) : r_src + (valid ? c - rank : 0);
          cp_async16(row + c, src, valid);
        }
      }
      cp_async_commit();
    };

    float o[RT][NT][4];
    float top[RT][2], sum[RT][2];     // running maxima of rows g and g + 8 of each tile (the same in every warp),
                                      // and this thread's share of the rows' sums (its own keys only)
#pragma unroll
    for (int tile = 0; tile < RT; ++tile) {
#pragma unroll
      for (int i = 0; i < NT; ++i) o[tile][i][0] = o[tile][i][1] = o[tile][i][2] = o[tile][i][3] = 0.f;
      top[tile][0] = top[tile][1] = -FLT_MAX;
      sum[tile][0] = sum[tile][1] = 0.f;
    }

    const int tiles = (end - begin + kTile - 1) / kTile;
    fetch(begin, 0);
    __syncthreads();
    copy(0);
    for (int i = 0; i < tiles; ++i) {
      const int buf = i & 1;
      const int base = begin + i * kTile;
      if (i + 1 < tiles) fetch(base + kTile, buf ^ 1);
      cp_async_wait<0>();
      __syncthreads();          // [A] tile i has landed; everybody is done with tile i - 1, the weights and the maxima
      if (i + 1 < tiles) copy(buf ^ 1);

      // scores of keys 8 * warp .. + 7 for the rows of every tile
      float s[RT][4];
      {
        // two chains of dependent products (even and odd steps of 16), joined at the end
        float s2[RT][4];
#pragma unroll
        for (int tile = 0; tile < RT; ++tile)
#pragma unroll
          for (int x = 0; x < 4; ++x) s[tile][x] = s2[tile][x] = 0.f;
        uint32_t a_at = q_at;
        uint32_t b_at = k_at + (uint32_t)buf * (kTile * ld * 2);
        int k0 = 0;
        for (; k0 + 32 <= lay.depth; k0 += 32, a_at += 64, b_at += 64) {
          uint32_t b0, b1, b2, b3;
          ldsm_x2_at(b0, b1, b_at);
          ldsm_x2_at(b2, b3, b_at + 32);
#pragma unroll
          for (int tile = 0; tile < RT; ++tile) {
            uint32_t a[4], a2[4];
            ldsm_x4_at(a, a_at + tile * (kRows * ld * 2));
            ldsm_x4_at(a2, a_at + tile * (kRows * ld * 2) + 32);
            mma_bf16(s[tile], a, b0, b1);
            mma_bf16(s2[tile], a2, b2, b3);
          }
        }
        if (k0 < lay.depth) {
          uint32_t b0, b1;
          ldsm_x2_at(b0, b1, b_at);
#pragma unroll
          for (int tile = 0; tile < RT; ++tile) {
            uint32_t a[4];
            ldsm_x4_at(a, a_at + tile * (kRows * ld * 2));
            mma_bf16(s[tile], a, b0, b1);
          }
        }
#pragma unroll
        for (int tile = 0; tile < RT; ++tile)
#pragma unroll
          for (int x = 0; x < 4; ++x) s[tile][x] += s2[tile][x];
      }
      const int key0 = base + warp * 8 + 2 * tg;
      bool in0[RT], in1[RT];
#pragma unroll
      for (int tile = 0; tile < RT; ++tile) {
        const int last = min(end - 1, position[tile]);      // the later token of a pair sees one key more
        in0[tile] = key0 <= last && key0 >= lowest[tile];
        in1[tile] = key0 + 1 <= last && key0 + 1 >= lowest[tile];
        s[tile][0] = in0[tile] ? s[tile][0] * scale : -FLT_MAX;
        s[tile][1] = in1[tile] ? s[tile][1] * scale : -FLT_MAX;
        s[tile][2] = in0[tile] ? s[tile][2] * scale : -FLT_MAX;
        s[tile][3] = in1[tile] ? s[tile][3] * scale : -FLT_MAX;
        const float top0 = quad_max(fmaxf(s[tile][0], s[tile][1])), top1 = quad_max(fmaxf(s[tile][2], s[tile][3]));
        if (tg == 0) {
          wmax[warp * ROWS + tile * kRows + g] = top0;
          wmax[warp * ROWS + tile * kRows + g + 8] = top1;
        }
      }
      __syncthreads();          // [B]
#pragma unroll
      for (int tile = 0; tile < RT; ++tile) {
        float new0 = top[tile][0], new1 = top[tile][1];
#pragma unroll
        for (int w = 0; w < kWarps; ++w) {
          new0 = fmaxf(new0, wmax[w * ROWS + tile * kRows + g]);
          new1 = fmaxf(new1, wmax[w * ROWS + tile * kRows + g + 8]);
        }
        const float fix0 = expf(top[tile][0] - new0), fix1 = expf(top[tile][1] - new1);
        top[tile][0] = new0;
        top[tile][1] = new1;
        const float p0 = in0[tile] ? expf(s[tile][0] - new0) : 0.f, p1 = in1[tile] ? expf(s[tile][1] - new0) : 0.f;
        const float p2 = in0[tile] ? expf(s[tile][2] - new1) : 0.f, p3 = in1[tile] ? expf(s[tile][3] - new1) : 0.f;
        sum[tile][0] = sum[tile][0] * fix0 + p0 + p1;
        sum[tile][1] = sum[tile][1] * fix1 + p2 + p3;
        // the weight as two bfloat16 terms: its rounding, and the rounding of what that left
        const __nv_bfloat162 hi_a = __floats2bfloat162_rn(p0, p1), hi_b = __floats2bfloat162_rn(p2, p3);
        const float2 fa = __bfloat1622float2(hi_a), fb = __bfloat1622float2(hi_b);
        const __nv_bfloat162 lo_a = __floats2bfloat162_rn(p0 - fa.x, p1 - fa.y), lo_b = __floats2bfloat162_rn(p2 - fb.x, p3 - fb.y);
        const int col = warp * 8 + 2 * tg;
        bf16* rows = ps + tile * kRows * PLD;
        *reinterpret_cast<__nv_bfloat162*>(rows + g * PLD + col) = hi_a;
        *reinterpret_cast<__nv_bfloat162*>(rows + (g + 8) * PLD + col) = hi_b;
        *reinterpret_cast<__nv_bfloat162*>(rows + ROWS * PLD + g * PLD + col) = lo_a;
        *reinterpret_cast<__nv_bfloat162*>(rows + ROWS * PLD + (g + 8) * PLD + col) = lo_b;
#pragma unroll
        for (int n = 0; n < NT; ++n) {
          o[tile][n][0] *= fix0;
          o[tile][n][1] *= fix0;
          o[tile][n][2] *= fix1;
          o[tile][n][3] *= fix1;
        }
      }
      __syncthreads();          // [C] all weights of the tile are in shared memory
      {
        uint32_t b_at = v_at + (uint32_t)buf * (kTile * ld * 2);
#pragma unroll
        for (int k0 = 0; k0 < kTile; k0 += 16, b_at += 16 * ld * 2) {
          uint32_t hi[RT][4], lo[RT][4];
#pragma unroll
          for (int tile = 0; tile < RT; ++tile) {
            ldsm_x4_at(hi[tile], p_at + (tile * kRows * PLD + k0) * 2);
            ldsm_x4_at(lo[tile], p_at + ((ROWS + tile * kRows) * PLD + k0) * 2);
          }
#pragma unroll
          for (int n = 0; n < NT; ++n) {
            uint32_t b0, b1;
            ldsm_x2_trans_at(b0, b1, b_at + n * 16);
#pragma unroll
            for (int tile = 0; tile < RT; ++tile) {
              mma_bf16(o[tile][n], hi[tile], b0, b1);
              mma_bf16(o[tile][n], lo[tile], b0, b1);
            }
          }
        }
      }
    }

    // the rows' sums: over the four threads of a quad, then over the warps
    __syncthreads();
#pragma unroll
    for (int tile = 0; tile < RT; ++tile) {
      const float l0 = quad_sum(sum[tile][0]), l1 = quad_sum(sum[tile][1]);
      if (tg == 0) {
        wsum[warp * ROWS + tile * kRows + g] = l0;
        wsum[warp * ROWS + tile * kRows + g + 8] = l1;
      }
    }
    __syncthreads();
#pragma unroll
    for (int tile = 0; tile < RT; ++tile) {
      const int t = token[tile];
      if (t < 0) continue;
      float total0 = 0.f, total1 = 0.f;
#pragma unroll
      for (int w = 0; w < kWarps; ++w) {
        total0 += wsum[w * ROWS + tile * kRows + g];
        total1 += wsum[w * ROWS + tile * kRows + g + 8];
      }
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const int h = h0 + g + 8 * half;
        if (h >= heads) continue;
        const float m = top[tile][half], l = half ? total1 : total0;
        if (ranges == 1) {
          float total = l, keep = 1.f;
          if (sink) {
            const float peak = fmaxf(m, sink[h]);
            keep = expf(m - peak);
            total = l * keep + expf(sink[h] - peak);
          }
          const float inv = keep / total;
          float* dst = out + ((size_t)t * heads + h) * rank;
#pragma unroll
          for (int n = 0; n < NT; ++n) {
            const int col = warp * CW + n * 8 + 2 * tg;
            if (col < rank) dst[col] = o[tile][n][2 * half] * inv;
            if (col + 1 < rank) dst[col + 1] = o[tile][n][2 * half + 1] * inv;
          }
        } else {
          float* share = part + (((size_t)t * heads + h) * ranges + blockIdx.z) * (rank + 2);
          if (warp == 0 && tg == 0) {
            share[0] = m;
            share[1] = l;
          }
#pragma unroll
          for (int n = 0; n < NT; ++n) {
            const int col = warp * CW + n * 8 + 2 * tg;
            if (col < rank) share[2 + col] = o[tile][n][2 * half];
            if (col + 1 < rank) share[2 + col + 1] = o[tile][n][2 * half + 1];
          }
        }
      }
    }
  }
}

}  // namespace cie

// 1 if the kernel takes these sizes (bfloat16 pages; latent and rotated part multiples of 8, latent up to 512).
extern "C" int cie_latent_attention_tensor_supports(int rank, int rot) {
  return rank % 8 == 0 && rot % 8 == 0 && rank >= 8 && rot >= 8 && rank <= 512 ? 1 : 0;
}

extern "C" int cie_latent_attention_tensor(const float* q_abs, const float* q_raw, int q_raw_stride, int q_raw_head,
                                           float* out, float* part, const void* c_pool, const void* r_pool,
                                           const int* positions, const int* request_of_token, const int* table,
                                           int table_width, int num_pages, const float* inv_freq, float magnitude,
                                           int interleaved, int rot_dims, const float* sink, int tokens, int heads,
                                           int rank, int rot, int page_size, float scale, int range_keys, int ranges,
                                           int pair_tokens, int window, int* err, void* stream) {
  using namespace cie;
  if (tokens <= 0) return 0;
  if (!cie_latent_attention_tensor_supports(rank, rot)) CIE_FAIL("latent_attention_tensor: sizes %d + %d", rank, rot);
  if (range_keys < kTile || range_keys % kTile) CIE_FAIL("latent_attention_tensor: key ranges are multiples of %d", kTile);
  if (ranges < 1 || ranges > 65535 || (ranges > 1 && !part)) CIE_FAIL("latent_attention_tensor: %d key ranges", ranges);
  const int nt = (rank + 63) / 64;
  // prompt portions (no key ranges, more than one token): two tokens a CTA, if shared memory has the room
  int row_tiles = (ranges == 1 && tokens > 1 && pair_tokens) ? 2 : 1;
  if (Layout::of(rank, rot, 8 * nt, row_tiles).bytes() > 220 * 1024) row_tiles = 1;
  const Layout lay = Layout::of(rank, rot, 8 * nt, row_tiles);
  const size_t smem = lay.bytes();
  if (smem > 220 * 1024) CIE_FAIL("latent_attention_tensor: %zu bytes of shared memory", smem);
  const dim3 grid((tokens + row_tiles - 1) / row_tiles, (heads + kRows - 1) / kRows, ranges);
#define CIE_LATENT_TENSOR_RT(NT, RT)                                                                                \
  {                                                                                                                 \
    static bool raised = false;                                                                                     \
    if (!raised) {                                                                                                  \
      if (cudaFuncSetAttribute(latent_attention_tensor_kernel<NT, RT>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                               220 * 1024) != cudaSuccess)                                                          \
        CIE_FAIL("latent_attention_tensor: cannot raise the shared memory limit");                                  \
      raised = true;                                                                                                \
    }                                                                                                               \
    CIE_LAUNCH("latent_attention_tensor", (latent_attention_tensor_kernel<NT, RT>), grid, dim3(kWarps * 32), smem,  \
               (cudaStream_t)stream, q_abs, q_raw, q_raw_stride, q_raw_head, out, part, (const bf16*)c_pool,        \
               (const bf16*)r_pool, positions, request_of_token, table, table_width, num_pages, inv_freq, magnitude, \
               interleaved, rot_dims, sink, tokens, heads, rank, rot, page_size, scale, range_keys, ranges, window, \
               err);                                                                                                \
  }
#define CIE_LATENT_TENSOR(NT)                        \
  if (row_tiles == 2) CIE_LATENT_TENSOR_RT(NT, 2)    \
  else CIE_LATENT_TENSOR_RT(NT, 1)
  switch (nt) {
    case 1: CIE_LATENT_TENSOR(1) break;
    case 2: CIE_LATENT_TENSOR(2) break;
    case 3: CIE_LATENT_TENSOR(3) break;
    case 4: CIE_LATENT_TENSOR(4) break;
    case 5: CIE_LATENT_TENSOR(5) break;
    case 6: CIE_LATENT_TENSOR(6) break;
    case 7: CIE_LATENT_TENSOR(7) break;
    default: CIE_LATENT_TENSOR(8) break;
  }
#undef CIE_LATENT_TENSOR
#undef CIE_LATENT_TENSOR_RT
  return 0;
}
