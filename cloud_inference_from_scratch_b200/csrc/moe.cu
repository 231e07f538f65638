// Routed experts (mixture of experts) for a flat batch of tokens:
//
//   route      router logits in float32 (token row times a float32 router matrix, plus a bias if one is
//              stored), a score function over all experts (softmax), the `top` largest of score +
//              correction, and as mixing weights the scores of the chosen experts (optionally renormalised
//              to sum 1); or (`chosen_softmax`) the `top` largest LOGITS and as weights the softmax over
//              those logits alone
//   plan       counts per expert -> offsets; every (token, choice) pair gets a place in its expert's
//              run of rows; runs are cut into tiles of 128 rows for the grouped products
//   gate_up    rows gathered by place, times the expert's stacked gate and up matrices, SiLU(gate)*up
//   down       times the expert's down matrix, written to the pair's own row (float32)
//   combine    y[t] = sum over the token's choices, in the order they were chosen, of weight * row
//
// The grouped products here run on the CUDA cores with float32 accumulation, one fused multiply-add
// per k in ascending order: the 32-bit path's products, and what every shape can fall back on.  A
// pair's row does not depend on which place it got, so the batch never changes a result.
#include "common.cuh"

#include <cfloat>

CIE_DEFINE_LAST_ERROR()

namespace cie {

constexpr int kMaxExperts = 1024;
constexpr int kRowTile = 128;         // rows of a tile of the grouped products

// ---------------------------------------------------------------- route
// One block of four warps per token: the token's row goes to shared memory as float32, the warps
// share the experts (a lane strides over the row with 16-byte loads of the router matrix where the
// row length allows), then the first warp turns logits into scores and chooses.
// ids / weights: [tokens][top]; counts[e] += 1 per choice.
constexpr int kRouteWarps = 8;
template <typename T>
__global__ void __launch_bounds__(kRouteWarps * 32)
moe_route_kernel(const T* __restrict__ x, const float* __restrict__ router,
                 const float* __restrict__ correction, int* __restrict__ ids,
                 float* __restrict__ weights, int* __restrict__ counts, int tokens,
                 int hidden, int experts, int top, int renormalize, const float* __restrict__ logit_bias,
                 int chosen_softmax) {
  extern __shared__ __align__(16) float score_s[];      // [2 * experts]: scores, then choice scores; then the row
  pdl_wait();
  pdl_trigger();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x;
  float* score = score_s;
  float* choice = score + experts;
  float* row_s = score_s + ((2 * experts + 3) & ~3);
  const T* row = x + (size_t)t * hidden;
  for (int k = threadIdx.x; k < hidden; k += blockDim.x) row_s[k] = to_float(row[k]);
  __syncthreads();
  const bool wide = hidden % 4 == 0;
  for (int e = warp; e < experts; e += kRouteWarps) {
    const float* w = router + (size_t)e * hidden;
    float dot = 0.f;
    if (wide) {
      // eight 16-byte loads of the router row are asked for before the first is used: the row comes
      // from memory once a step and nothing else hides that trip
      for (int k0 = 4 * lane; k0 < hidden; k0 += 8 * 128) {
        float4 wv[8];
#pragma unroll
        for (int u = 0; u < 8; ++u)
          wv[u] = k0 + 128 * u < hidden ? *reinterpret_cast<const float4*>(w + k0 + 128 * u) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          if (k0 + 128 * u >= hidden) break;
          const float4 xv = *reinterpret_cast<const float4*>(row_s + k0 + 128 * u);
          dot = fmaf(xv.x, wv[u].x, dot);
          dot = fmaf(xv.y, wv[u].y, dot);
          dot = fmaf(xv.z, wv[u].z, dot);
          dot = fmaf(xv.w, wv[u].w, dot);
        }
      }
    } else {
      for (int k = lane; k < hidden; k += 32) dot = fmaf(row_s[k], w[k], dot);
    }
    dot = warp_sum(dot);
    if (lane == 0) score[e] = logit_bias ? dot + logit_bias[e] : dot;
  }
  __syncthreads();
  if (warp != 0) return;
  __syncwarp();
  if (chosen_softmax) {
    // the largest logits win (lowest index on ties); their weights are exp(z - z_first) over the sum of those
    for (int e = lane; e < experts; e += 32) choice[e] = score[e];
    __syncwarp();
    float first = 0.f, total = 0.f, mine = 0.f;
    for (int j = 0; j < top; ++j) {
      float best = -FLT_MAX;
      int best_e = experts;
      for (int e = lane; e < experts; e += 32)
        if (choice[e] > best) { best = choice[e]; best_e = e; }
      for (int offset = 16; offset > 0; offset >>= 1) {
        const float other = __shfl_xor_sync(0xffffffffu, best, offset);
        const int other_e = __shfl_xor_sync(0xffffffffu, best_e, offset);
        if (other > best || (other == best && other_e < best_e)) { best = other; best_e = other_e; }
      }
      if (j == 0) first = best;
      const float w = expf(best - first);
      total += w;
      if (lane == j) mine = w;
      if (lane == 0) {
        ids[(size_t)t * top + j] = best_e;
        choice[best_e] = -FLT_MAX;
        atomicAdd(counts + best_e, 1);
      }
      __syncwarp();
    }
    if (lane < top) weights[(size_t)t * top + lane] = mine / total;
    return;
  }
  float m = -FLT_MAX;
  for (int e = lane; e < experts; e += 32) m = fmaxf(m, score[e]);
  m = warp_max(m);
  float sum = 0.f;
  for (int e = lane; e < experts; e += 32) sum += expf(score[e] - m);
  sum = warp_sum(sum);
  for (int e = lane; e < experts; e += 32) {
    const float s = expf(score[e] - m) / sum;
    score[e] = s;
    choice[e] = s + (correction ? correction[e] : 0.f);
  }
  __syncwarp();
  float chosen_sum = 0.f;
  for (int j = 0; j < top; ++j) {
    float best = -FLT_MAX;
    int best_e = experts;
    for (int e = lane; e < experts; e += 32)
      if (choice[e] > best) { best = choice[e]; best_e = e; }
    // largest value, lowest index on ties
    for (int offset = 16; offset > 0; offset >>= 1) {
      const float other = __shfl_xor_sync(0xffffffffu, best, offset);
      const int other_e = __shfl_xor_sync(0xffffffffu, best_e, offset);
      if (other > best || (other == best && other_e < best_e)) { best = other; best_e = other_e; }
    }
    if (lane == 0) {
      ids[(size_t)t * top + j] = best_e;
      weights[(size_t)t * top + j] = score[best_e];
      choice[best_e] = -FLT_MAX;
      atomicAdd(counts + best_e, 1);
    }
    chosen_sum += score[best_e];
    __syncwarp();
  }
  if (renormalize && lane < top) weights[(size_t)t * top + lane] /= chosen_sum;
}

// ---------------------------------------------------------------- plan
// One block.  offsets[e] = first place of expert e (offsets[experts] = pairs); place_to_pair[p] =
// the (token, choice) pair at place p; tiles: (expert, first place, rows) per tile, tile_count[0].
__global__ void moe_plan_kernel(const int* __restrict__ ids, const int* __restrict__ counts,
                                int* __restrict__ offsets, int* __restrict__ cursors,
                                int* __restrict__ place_to_pair, int* __restrict__ tiles,
                                int* __restrict__ tile_count, int pairs, int experts) {
  __shared__ int off_s[kMaxExperts + 1];
  __shared__ int tile_s[kMaxExperts + 1];
  pdl_wait();
  pdl_trigger();
  if (threadIdx.x == 0) {
    int total = 0, tile_total = 0;
    for (int e = 0; e < experts; ++e) {
      off_s[e] = total;
      tile_s[e] = tile_total;
      total += counts[e];
      tile_total += (counts[e] + kRowTile - 1) / kRowTile;
    }
    off_s[experts] = total;
    tile_s[experts] = tile_total;
    tile_count[0] = tile_total;
  }
  __syncthreads();
  for (int e = threadIdx.x; e <= experts; e += blockDim.x) {
    offsets[e] = off_s[e];
    if (e < experts) {
      cursors[e] = 0;
      const int n = off_s[e + 1] - off_s[e];
      for (int j = 0, tile = tile_s[e]; j < n; j += kRowTile, ++tile) {
        tiles[3 * tile] = e;
        tiles[3 * tile + 1] = off_s[e] + j;
        tiles[3 * tile + 2] = min(kRowTile, n - j);
      }
    }
  }
  __syncthreads();
  for (int pair = threadIdx.x; pair < pairs; pair += blockDim.x) {
    const int e = ids[pair];
    place_to_pair[off_s[e] + atomicAdd(cursors + e, 1)] = pair;
  }
}

// ---------------------------------------------------------------- grouped products (CUDA cores)
// Block y of the grid takes half (64 rows) of tile y / 2 of the plan (blocks beyond tile_count leave
// at once).
//   kGateUp  A row p = x[place_to_pair[p] / top]; W = w_gate[e], w_up[e] ([ff][hidden] each);
//            out[p][n] = SiLU(a.gate_n) * (a.up_n), activation type, rows by place
//   else     A row p = act[p]; W = w_down[e] ([hidden][ff]); out[place_to_pair[p]][n], float32
template <typename T, bool kGateUp>
__global__ void __launch_bounds__(256)
moe_grouped_simt_kernel(const T* __restrict__ a, const T* __restrict__ w0, const T* __restrict__ w1,
                        void* __restrict__ out, const int* __restrict__ place_to_pair,
                        const int* __restrict__ tiles, const int* __restrict__ tile_count, int top,
                        int n_total, int k_total) {
  constexpr int kTileN = 64, kTileK = 16, kHalf = 64;
  static_assert(kRowTile == 2 * kHalf, "a block takes half a tile");
  __shared__ float a_tile[kTileK][kHalf + 4];
  __shared__ float w_tile[kGateUp ? 2 : 1][kTileK][kTileN + 4];
  __shared__ int src_row[kHalf];
  pdl_wait();
  pdl_trigger();
  const int tile = blockIdx.y >> 1, half = blockIdx.y & 1;
  if (tile >= tile_count[0]) return;
  const int expert = tiles[3 * tile], place0 = tiles[3 * tile + 1] + kHalf * half, rows = tiles[3 * tile + 2] - kHalf * half;
  if (rows <= 0) return;
  const int tid = threadIdx.x;
  if (tid < kHalf) {
    int r = -1;
    if (tid < rows) r = kGateUp ? place_to_pair[place0 + tid] / top : place0 + tid;
    src_row[tid] = r;
  }
  __syncthreads();
  const int n0 = blockIdx.x * kTileN;
  const T* wg = w0 + (size_t)expert * n_total * k_total;
  const T* wu = kGateUp ? w1 + (size_t)expert * n_total * k_total : nullptr;
  const int tm = (tid / 16) * 4, tn = (tid % 16) * 4;
  float acc[4][4] = {}, acc_up[kGateUp ? 4 : 1][4] = {};
  for (int k0 = 0; k0 < k_total; k0 += kTileK) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int e = tid + i * 256;
      const int r = e / kTileK, kk = e % kTileK;
      const int gk = k0 + kk, gn = n0 + r;
      const int row = src_row[r];
      a_tile[kk][r] = (row >= 0 && gk < k_total) ? to_float(a[(size_t)row * k_total + gk]) : 0.f;
      const bool in = gn < n_total && gk < k_total;
      w_tile[0][kk][r] = in ? to_float(wg[(size_t)gn * k_total + gk]) : 0.f;
      if constexpr (kGateUp) w_tile[1][kk][r] = in ? to_float(wu[(size_t)gn * k_total + gk]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < kTileK; ++kk) {
      float av[4], wv[4], uv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) av[i] = a_tile[kk][tm + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        wv[j] = w_tile[0][kk][tn + j];
        if constexpr (kGateUp) uv[j] = w_tile[1][kk][tn + j];
      }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          acc[i][j] = fmaf(av[i], wv[j], acc[i][j]);
          if constexpr (kGateUp) acc_up[i][j] = fmaf(av[i], uv[j], acc_up[i][j]);
        }
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = tm + i;
    if (r >= rows) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int gn = n0 + tn + j;
      if (gn >= n_total) continue;
      if constexpr (kGateUp) {
        const float g = acc[i][j];
        reinterpret_cast<T*>(out)[(size_t)(place0 + r) * n_total + gn] =
            from_float<T>(g / (1.f + expf(-g)) * acc_up[i][j]);
      } else {
        reinterpret_cast<float*>(out)[(size_t)place_to_pair[place0 + r] * n_total + gn] = acc[i][j];
      }
    }
  }
}

// ---------------------------------------------------------------- grouped products (tensor cores)
// bfloat16 operands, float32 accumulators, mma.sync m16n8k16.  A tile is 128 rows of one expert by
// 64 output columns (gate_up: the 64 gate columns AND their 64 up columns, so that a thread ends
// with both halves of SiLU(gate) * up); K advances in steps of 32 through a four-stage cp.async
// ring.  Eight warps: four along the rows, two along the columns.  Rows are gathered by place;
// rows and columns beyond the edges are zero-filled by the copy and never stored.
__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool valid) {
  const unsigned d = (unsigned)__cvta_generic_to_shared(dst);
  const int bytes = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void ldmatrix_x4(unsigned (&r)[4], const void* p) {
  const unsigned a = (unsigned)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

constexpr int kTcStages = 4, kTcK = 32, kTcPad = 8, kTcCols = 64;
constexpr int kTcLd = kTcK + kTcPad;                      // 40 elements = 80 bytes a row: ldmatrix without conflicts

template <bool kGateUp>
constexpr size_t moe_tc_smem() {
  return (size_t)kTcStages * (kRowTile + (kGateUp ? 2 : 1) * kTcCols) * kTcLd * sizeof(__nv_bfloat16);
}

template <bool kGateUp>
__global__ void __launch_bounds__(256)
moe_grouped_tc_kernel(const __nv_bfloat16* __restrict__ a, const __nv_bfloat16* __restrict__ w0,
                      const __nv_bfloat16* __restrict__ w1, void* __restrict__ out,
                      const int* __restrict__ place_to_pair, const int* __restrict__ tiles,
                      const int* __restrict__ tile_count, int top, int n_total, int k_total, int interleaved) {
  // interleaved (gate_up only): w0 holds [experts][2 * n_total][k], 16 gate rows, their 16 up rows, ...
  constexpr int kWRows = kGateUp ? 2 * kTcCols : kTcCols;
  constexpr int kNT = kGateUp ? 8 : 4;                    // 8-column accumulators of a warp
  extern __shared__ __align__(16) unsigned char tc_smem[];
  typedef __nv_bfloat16 (*ATile)[kRowTile][kTcLd];
  typedef __nv_bfloat16 (*WTile)[kWRows][kTcLd];
  ATile a_s = reinterpret_cast<ATile>(tc_smem);
  WTile w_s = reinterpret_cast<WTile>(tc_smem + (size_t)kTcStages * kRowTile * kTcLd * sizeof(__nv_bfloat16));
  __shared__ int src_row[kRowTile];
  __shared__ int dst_row[kRowTile];
  pdl_wait();
  pdl_trigger();
  if ((int)blockIdx.y >= tile_count[0]) return;
  const int expert = tiles[3 * blockIdx.y], place0 = tiles[3 * blockIdx.y + 1], rows = tiles[3 * blockIdx.y + 2];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid < kRowTile) {
    int src = -1, dst = -1;
    if (tid < rows) {
      const int pair = place_to_pair[place0 + tid];
      src = kGateUp ? pair / top : place0 + tid;
      dst = kGateUp ? place0 + tid : pair;
    }
    src_row[tid] = src;
    dst_row[tid] = dst;
  }
  __syncthreads();
  const int n0 = blockIdx.x * kTcCols;
  const __nv_bfloat16* wg = w0 + (size_t)expert * (interleaved ? 2 : 1) * n_total * k_total;
  const __nv_bfloat16* wu = (kGateUp && !interleaved) ? w1 + (size_t)expert * n_total * k_total : nullptr;
  const int k_steps = (k_total + kTcK - 1) / kTcK;

  auto load_stage = [&](int stage, int step) {
    const int k0 = step * kTcK;
    const int c = (tid & 3) * 8;
#pragma unroll
    for (int i = 0; i < kRowTile / 64; ++i) {       // A: 128 rows x 4 pieces of 8 elements
      const int r = (tid >> 2) + i * 64;
      const int row = src_row[r];
      const bool ok = row >= 0 && k0 + c < k_total;
      cp_async16(&a_s[stage][r][c], ok ? a + (size_t)row * k_total + k0 + c : a, ok);
    }
#pragma unroll
    for (int i = 0; i < kWRows / 64; ++i) {
      const int r = (tid >> 2) + i * 64;
      const bool up = kGateUp && r >= kTcCols;
      const int gn = n0 + (up ? r - kTcCols : r);
      const bool ok = gn < n_total && k0 + c < k_total;
      const __nv_bfloat16* base = (up && !interleaved) ? wu : wg;
      const size_t w_row = interleaved ? (size_t)(gn >> 4) * 32 + (gn & 15) + (up ? 16 : 0) : (size_t)gn;
      cp_async16(&w_s[stage][r][c], ok ? base + w_row * k_total + k0 + c : wg, ok);
    }
  };

  const int wm = warp >> 1, wn = warp & 1;        // rows 32 * wm .., columns 32 * wn .. (of gate and of up)
  float acc[2][kNT][4] = {};
#pragma unroll
  for (int s = 0; s < kTcStages - 1; ++s) {
    if (s < k_steps) load_stage(s, s);
    cp_async_commit();
  }
  for (int step = 0; step < k_steps; ++step) {
    cp_async_wait<kTcStages - 2>();
    __syncthreads();
    const int next = step + kTcStages - 1;
    if (next < k_steps) load_stage(next % kTcStages, next);
    cp_async_commit();
    const int stage = step % kTcStages;
#pragma unroll
    for (int kk = 0; kk < kTcK; kk += 16) {
      unsigned af[2][4];
#pragma unroll
      for (int mt = 0; mt < 2; ++mt)
        ldmatrix_x4(af[mt], &a_s[stage][32 * wm + 16 * mt + (lane & 15)][kk + (lane >> 4) * 8]);
      // a load gives two accumulators' worth (16 columns): rows (lane & 7) + 8 * (lane >> 4), k half (lane >> 3) & 1
#pragma unroll
      for (int nb = 0; nb < kNT / 2; ++nb) {
        const int w_row = (nb >= 2 ? kTcCols + 16 * (nb - 2) : 16 * nb) + 32 * wn;
        unsigned bf[4];
        ldmatrix_x4(bf, &w_s[stage][w_row + (lane & 7) + ((lane >> 4) << 3)][kk + ((lane >> 3) & 1) * 8]);
#pragma unroll
        for (int mt = 0; mt < 2; ++mt) {
          mma_bf16(acc[mt][2 * nb], af[mt], bf[0], bf[1]);
          mma_bf16(acc[mt][2 * nb + 1], af[mt], bf[2], bf[3]);
        }
      }
    }
  }
  cp_async_wait<0>();
#pragma unroll
  for (int mt = 0; mt < 2; ++mt)
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int r = 32 * wm + 16 * mt + (lane >> 2) + 8 * half;
      const int dst = dst_row[r];
      if (dst < 0) continue;
#pragma unroll
      for (int nt = 0; nt < 4; ++nt)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int gn = n0 + 32 * wn + 8 * nt + (lane & 3) * 2 + e;
          if (gn >= n_total) continue;
          if constexpr (kGateUp) {
            const float g = acc[mt][nt][2 * half + e], u = acc[mt][4 + nt][2 * half + e];
            reinterpret_cast<__nv_bfloat16*>(out)[(size_t)dst * n_total + gn] = __float2bfloat16_rn(g / (1.f + expf(-g)) * u);
          } else {
            reinterpret_cast<float*>(out)[(size_t)dst * n_total + gn] = acc[mt][nt][2 * half + e];
          }
        }
    }
}

// y[t][i] = sum_j weights[t][j] * rows[t * top + j][i], j ascending; float32 or activation type out.
template <typename TOut>
__global__ void moe_combine_kernel(const float* __restrict__ rows, const float* __restrict__ weights,
                                   TOut* __restrict__ y, int hidden, int top) {
  pdl_wait();
  pdl_trigger();
  const int t = blockIdx.x;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    float total = 0.f;
    for (int j = 0; j < top; ++j)
      total = fmaf(weights[(size_t)t * top + j], rows[((size_t)t * top + j) * hidden + i], total);
    y[(size_t)t * hidden + i] = from_float<TOut>(total);
  }
}

}  // namespace cie

using namespace cie;

extern "C" int cie_moe_row_tile() { return kRowTile; }

// counts, offsets (experts + 1), cursors, tile_count (1) and tiles (3 * (pairs / 64 + experts)) are
// int32 scratch of the caller; counts is zeroed here.
extern "C" int cie_moe_route(const void* x, const float* router, const float* correction, int* ids,
                             float* weights, int* counts, int* offsets, int* cursors, int* place_to_pair,
                             int* tiles, int* tile_count, int tokens, int hidden, int experts, int top,
                             int renormalize, const float* logit_bias, int chosen_softmax, int dtype, void* stream) {
  if (tokens <= 0) return 0;
  if (experts < 1 || experts > kMaxExperts) CIE_FAIL("moe_route: 1..%d experts, got %d", kMaxExperts, experts);
  if (top < 1 || top > experts || top > 32) CIE_FAIL("moe_route: top %d of %d experts (at most 32)", top, experts);
  cudaStream_t s = (cudaStream_t)stream;
  if (cudaMemsetAsync(counts, 0, sizeof(int) * experts, s) != cudaSuccess) CIE_FAIL("moe_route: memset failed");
  const int warps = kRouteWarps;
  const size_t smem = (size_t)(((2 * experts + 3) & ~3) + hidden) * sizeof(float);
  if (smem > 200 * 1024) CIE_FAIL("moe_route: a row of %d elements does not fit shared memory", hidden);
  const int blocks = tokens;
  if (dtype == kFloat32) {
    if (smem > 48 * 1024 && cudaFuncSetAttribute(moe_route_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
      CIE_FAIL("moe_route: cannot reserve %zu bytes of shared memory", smem);
    CIE_LAUNCH("moe_route", moe_route_kernel<float>, dim3(blocks), dim3(warps * 32), smem, s, (const float*)x, router,
               correction, ids, weights, counts, tokens, hidden, experts, top, renormalize, logit_bias, chosen_softmax);
  } else if (dtype == kBFloat16) {
    if (smem > 48 * 1024 && cudaFuncSetAttribute(moe_route_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
      CIE_FAIL("moe_route: cannot reserve %zu bytes of shared memory", smem);
    CIE_LAUNCH("moe_route", moe_route_kernel<__nv_bfloat16>, dim3(blocks), dim3(warps * 32), smem, s,
               (const __nv_bfloat16*)x, router, correction, ids, weights, counts, tokens, hidden, experts, top,
               renormalize, logit_bias, chosen_softmax);
  } else {
    CIE_FAIL("moe_route: unknown element type code %d", dtype);
  }
  CIE_LAUNCH("moe_plan", moe_plan_kernel, dim3(1), dim3(1024), 0, s, ids, counts, offsets, cursors, place_to_pair,
             tiles, tile_count, tokens * top, experts);
  return 0;
}

// act: [pairs][ff] activation type, rows by place.  w_gate, w_up: [experts][ff][hidden].
extern "C" int cie_moe_gate_up_simt(const void* x, const void* w_gate, const void* w_up, void* act,
                                    const int* place_to_pair, const int* tiles, const int* tile_count,
                                    int tokens, int top, int experts, int ff, int hidden, int dtype,
                                    void* stream) {
  if (tokens <= 0) return 0;
  const int max_tiles = (tokens * top + kRowTile - 1) / kRowTile + experts;
  dim3 grid((ff + 63) / 64, 2 * max_tiles);
  if (dtype == kFloat32) {
    CIE_LAUNCH("moe_gate_up", (moe_grouped_simt_kernel<float, true>), grid, dim3(256), 0, (cudaStream_t)stream,
               (const float*)x, (const float*)w_gate, (const float*)w_up, act, place_to_pair, tiles, tile_count, top,
               ff, hidden);
  } else if (dtype == kBFloat16) {
    CIE_LAUNCH("moe_gate_up", (moe_grouped_simt_kernel<__nv_bfloat16, true>), grid, dim3(256), 0, (cudaStream_t)stream,
               (const __nv_bfloat16*)x, (const __nv_bfloat16*)w_gate, (const __nv_bfloat16*)w_up, act, place_to_pair,
               tiles, tile_count, top, ff, hidden);
  } else {
    CIE_FAIL("moe_gate_up: unknown element type code %d", dtype);
  }
  return 0;
}

// rows: float32 [pairs][hidden], row of pair (t, j) at t * top + j.  w_down: [experts][hidden][ff].
extern "C" int cie_moe_down_simt(const void* act, const void* w_down, float* rows, const int* place_to_pair,
                                 const int* tiles, const int* tile_count, int tokens, int top, int experts,
                                 int ff, int hidden, int dtype, void* stream) {
  if (tokens <= 0) return 0;
  const int max_tiles = (tokens * top + kRowTile - 1) / kRowTile + experts;
  dim3 grid((hidden + 63) / 64, 2 * max_tiles);
  if (dtype == kFloat32) {
    CIE_LAUNCH("moe_down", (moe_grouped_simt_kernel<float, false>), grid, dim3(256), 0, (cudaStream_t)stream,
               (const float*)act, (const float*)w_down, (const float*)nullptr, (void*)rows, place_to_pair, tiles,
               tile_count, top, hidden, ff);
  } else if (dtype == kBFloat16) {
    CIE_LAUNCH("moe_down", (moe_grouped_simt_kernel<__nv_bfloat16, false>), grid, dim3(256), 0, (cudaStream_t)stream,
               (const __nv_bfloat16*)act, (const __nv_bfloat16*)w_down, (const __nv_bfloat16*)nullptr, (void*)rows,
               place_to_pair, tiles, tile_count, top, hidden, ff);
  } else {
    CIE_FAIL("moe_down: unknown element type code %d", dtype);
  }
  return 0;
}

// The same two products on the tensor cores: bfloat16 only, hidden and ff multiples of 8, pointers
// aligned to 16 bytes (the caller checks).
// w_up null: w_gate holds both, [experts][2 ff][hidden], interleaved in blocks of 16 rows.
extern "C" int cie_moe_gate_up_tc(const void* x, const void* w_gate, const void* w_up, void* act,
                                  const int* place_to_pair, const int* tiles, const int* tile_count,
                                  int tokens, int top, int experts, int ff, int hidden, void* stream) {
  if (!w_up && ff % 16) CIE_FAIL("moe_gate_up_tc: interleaved weights need a multiple of 16 channels, got %d", ff);
  if (tokens <= 0) return 0;
  if (hidden % 8 || ff % 8) CIE_FAIL("moe_gate_up_tc: sizes %d / %d are no multiples of 8", hidden, ff);
  const int max_tiles = (tokens * top + kRowTile - 1) / kRowTile + experts;
  dim3 grid((ff + kTcCols - 1) / kTcCols, max_tiles);
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(moe_grouped_tc_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)moe_tc_smem<true>()) != cudaSuccess)
      CIE_FAIL("moe_gate_up_tc: cannot reserve %zu bytes of shared memory", moe_tc_smem<true>());
    configured = true;
  }
  CIE_LAUNCH("moe_gate_up_tc", moe_grouped_tc_kernel<true>, grid, dim3(256), moe_tc_smem<true>(), (cudaStream_t)stream,
             (const __nv_bfloat16*)x, (const __nv_bfloat16*)w_gate, (const __nv_bfloat16*)w_up, act, place_to_pair,
             tiles, tile_count, top, ff, hidden, w_up ? 0 : 1);
  return 0;
}

extern "C" int cie_moe_down_tc(const void* act, const void* w_down, float* rows, const int* place_to_pair,
                               const int* tiles, const int* tile_count, int tokens, int top, int experts,
                               int ff, int hidden, void* stream) {
  if (tokens <= 0) return 0;
  if (hidden % 8 || ff % 8) CIE_FAIL("moe_down_tc: sizes %d / %d are no multiples of 8", hidden, ff);
  const int max_tiles = (tokens * top + kRowTile - 1) / kRowTile + experts;
  dim3 grid((hidden + kTcCols - 1) / kTcCols, max_tiles);
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(moe_grouped_tc_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)moe_tc_smem<false>()) != cudaSuccess)
      CIE_FAIL("moe_down_tc: cannot reserve %zu bytes of shared memory", moe_tc_smem<false>());
    configured = true;
  }
  CIE_LAUNCH("moe_down_tc", moe_grouped_tc_kernel<false>, grid, dim3(256), moe_tc_smem<false>(), (cudaStream_t)stream,
             (const __nv_bfloat16*)act, (const __nv_bfloat16*)w_down, (const __nv_bfloat16*)nullptr, (void*)rows,
             place_to_pair, tiles, tile_count, top, hidden, ff, 0);
  return 0;
}

// y: [tokens][hidden], float32 (out_dtype 0) or bfloat16 (1).
extern "C" int cie_moe_combine(const float* rows, const float* weights, void* y, int tokens, int hidden,
                               int top, int out_dtype, void* stream) {
  if (tokens <= 0) return 0;
  int threads = 32;
  while (threads < hidden / 4 && threads < 1024) threads <<= 1;
  if (out_dtype == kFloat32) {
    CIE_LAUNCH("moe_combine", moe_combine_kernel<float>, dim3(tokens), dim3(threads), 0, (cudaStream_t)stream, rows,
               weights, (float*)y, hidden, top);
  } else if (out_dtype == kBFloat16) {
    CIE_LAUNCH("moe_combine", moe_combine_kernel<__nv_bfloat16>, dim3(tokens), dim3(threads), 0, (cudaStream_t)stream,
               rows, weights, (__nv_bfloat16*)y, hidden, top);
  } else {
    CIE_FAIL("moe_combine: unknown element type code %d", out_dtype);
  }
  return 0;
}
